"""Records what mxinO/holon's own CPU model computes on two tiny random Qwen3 models.

Run once, by hand, on a machine that has the reference checkout:

    python tests/golden/make_golden.py /path/to/holon

It imports holon's model code (recipe, units, CPU oracle kernels) from that checkout, builds the model without any
state so that it attends over whole sequences, and writes `tests/golden/qwen3_tiny.safetensors`: the logits of
every position of a few prompts. The weights are not stored: `tiny_weights` below makes them again from the seed,
and a checksum of them is stored so that a changed random generator shows as a skipped test, not a wrong one.
`tests/test_plain.py` compares `tests/plain_qwen3.py` with these logits.
"""
from __future__ import annotations

import json
import pathlib
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent

CONFIGS = {
    "a": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128),
    "b": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
              num_key_value_heads=1, head_dim=32, intermediate_size=160, vocab_size=384, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512),
}
PROMPT_LENGTHS = {"a": (5, 17), "b": (1, 9, 40)}
SEEDS = {"a": 0, "b": 1}


def tiny_weights(config, seed):
    """{HF name: float32 tensor}: matrices N(0, 0.02), norm weights 1 + N(0, 0.1), from one seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    h, d, inter = config["hidden_size"], config["head_dim"], config["intermediate_size"]
    hq, hkv = config["num_attention_heads"], config["num_key_value_heads"]

    def matrix(*shape):
        return torch.randn(*shape, generator=g) * 0.02

    def gain(n):
        return 1 + torch.randn(n, generator=g) * 0.1

    w = {"model.embed_tokens.weight": matrix(config["vocab_size"], h), "model.norm.weight": gain(h)}
    if not config["tie_word_embeddings"]:
        w["lm_head.weight"] = matrix(config["vocab_size"], h)
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"], w[p + "post_attention_layernorm.weight"] = gain(h), gain(h)
        w[p + "self_attn.q_proj.weight"] = matrix(hq * d, h)
        w[p + "self_attn.k_proj.weight"] = matrix(hkv * d, h)
        w[p + "self_attn.v_proj.weight"] = matrix(hkv * d, h)
        w[p + "self_attn.o_proj.weight"] = matrix(h, hq * d)
        w[p + "self_attn.q_norm.weight"], w[p + "self_attn.k_norm.weight"] = gain(d), gain(d)
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = matrix(inter, h), matrix(inter, h)
        w[p + "mlp.down_proj.weight"] = matrix(h, inter)
    return w


def prompts(name):
    g = torch.Generator().manual_seed(100 + SEEDS[name])
    return [torch.randint(0, CONFIGS[name]["vocab_size"], (n,), generator=g).tolist() for n in PROMPT_LENGTHS[name]]


def checksum(weights) -> float:
    return float(sum(t.double().abs().sum() for t in weights.values()))


def main(reference: pathlib.Path) -> None:
    from safetensors.torch import save_file
    for p in ("core", "std", "plugins", "testing"):
        sys.path.insert(0, str(reference / p))
    from holon.api import Manifest
    from holon.core.build import BuildContext, StepContext, build_model, load_weights
    from holon.core.plugins import Installed, PluginSet

    installed = {}
    for root in (reference / "std" / "holon_std", reference / "plugins" / "holon_plugins",
                 reference / "testing" / "holon_testing"):
        for toml in root.rglob("plugin.toml"):
            if "vendor" in toml.parts:
                continue
            m = Manifest.load(toml)
            installed[m.name] = Installed(m, ".".join(toml.parent.relative_to(root.parent).parts), toml.parent)
    plugins = PluginSet(installed)
    out = {}
    for name, config in CONFIGS.items():
        weights = tiny_weights(config, SEEDS[name])
        spec = plugins.load("models.qwen3").recipe(config, "hf_safetensors")
        ctx = BuildContext(plugins, torch.device("cpu"), torch.float32)
        model = build_model(spec, ctx)
        load_weights(model, ctx, list(weights.items()))
        ids = prompts(name)
        with torch.no_grad():
            logits = model(StepContext.whole_sequences(ids, "cpu"))
        out[f"{name}.logits"] = logits.float().contiguous()
        out[f"{name}.checksum"] = torch.tensor([checksum(weights)], dtype=torch.float64)
    save_file(out, str(HERE / "qwen3_tiny.safetensors"), metadata={"made_by": "tests/golden/make_golden.py",
                                                                  "configs": json.dumps(CONFIGS)})
    print({k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main(pathlib.Path(sys.argv[1]))

"""Records what mxinO/holon's own engine and sampler produce on the CPU, for the tests of sampling and scheduling.

Run once, by hand, on a machine that has the reference checkout:

    python tests/golden/make_engine_golden.py /path/to/holon

It imports the reference from that checkout (core, std, plugins and the test-only CPU oracle kernels), builds its
plugin set from the `plugin.toml` manifests, and writes `tests/golden/qwen3_tiny_engine.json`:

- `uniform`: the sampler's uniform of (seed, position) for a grid of seeds (below and above 2^32) and positions
  (std/holon_std/sampling/sampler.py:33-40);
- `draws`: for seeded random logits rows at temperature 0.7 and 1.3, the token the sampler's inverse-CDF draw picks with
  the uniform of (seed, position) (sampler.py:57-61, 137-146; the unfiltered path, which draws in vocabulary order);
- `engine`: the token ids the reference's `Engine.generate` returns on the two tiny models of `make_golden.py`, in
  float32 with its CPU oracle kernels: model "a" greedy (prompts of 5, 17 and 31 tokens, 16 tokens each, pages of 4)
  and model "b" at temperature 0.7 with seeds 11, 12, 13, 14 (prompts of 1, 9, 40 and 77 tokens, portions of 8 beside
  decoding requests, pages of 16, 12 tokens each), each also in a pool so small that requests are preempted.

The weights are those of `make_golden.tiny_weights`; their checksum is stored so that another random generator shows
as a skipped test. `tests/test_plain.py`, `tests/test_engine_cpu.py` and `tests/test_gpu_engine.py` compare the plain
implementation, the plain kernel table and the engine with this file.
"""
from __future__ import annotations

import json
import pathlib
import sys
import tempfile

import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import make_golden  # noqa: E402

SEEDS = (0, 1, 11, 12345, 2**31 + 7, 2**32 + 5, 2**40 + 99, 2**63 - 1)
POSITIONS = (0, 1, 2, 17, 255, 256, 4096, 2**20 + 3)
WORKLOADS = {
    "a": dict(lengths=(5, 17, 31), temperature=0.0, seeds=(0, 0, 0), max_tokens=16, page_size=4, chunk_with_decode=8,
              max_step_tokens=32, max_seqs=4, max_model_len=64),
    "b": dict(lengths=(1, 9, 40, 77), temperature=0.7, seeds=(11, 12, 13, 14), max_tokens=12, page_size=16,
              chunk_with_decode=8, max_step_tokens=16, max_seqs=4, max_model_len=128),
}
DRAW_ROWS, DRAW_VOCAB = 6, 389


def workload_prompts(name):
    g = torch.Generator().manual_seed(300 + make_golden.SEEDS[name])
    vocab = make_golden.CONFIGS[name]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in WORKLOADS[name]["lengths"]]


def draw_logits():
    g = torch.Generator().manual_seed(77)
    return torch.randn(DRAW_ROWS, DRAW_VOCAB, generator=g) * 2.0


def main(reference: pathlib.Path) -> None:
    from safetensors.torch import save_file
    for p in ("core", "std", "plugins", "testing"):
        sys.path.insert(0, str(reference / p))
    from holon.api import Manifest, SamplingParams
    from holon.core.engine import Engine, EngineConfig
    from holon.core.plugins import Installed, PluginSet
    from holon_std.sampling import sampler

    installed = {}
    for root in (reference / "std" / "holon_std", reference / "plugins" / "holon_plugins",
                 reference / "testing" / "holon_testing"):
        for toml in root.rglob("plugin.toml"):
            if "vendor" in toml.parts:
                continue
            m = Manifest.load(toml)
            installed[m.name] = Installed(m, ".".join(toml.parent.relative_to(root.parent).parts), toml.parent)
    plugins = PluginSet(installed)

    out = {"made_by": "tests/golden/make_engine_golden.py", "seeds": list(SEEDS), "positions": list(POSITIONS)}
    seeds = torch.tensor([s for s in SEEDS for _ in POSITIONS], dtype=torch.int64)
    positions = torch.tensor([p for _ in SEEDS for p in POSITIONS], dtype=torch.int64)
    out["uniform"] = [float(u) for u in sampler.uniform(seeds, positions).double()]

    logits = draw_logits()
    draws = []
    for temperature in (0.7, 1.3):
        for seed in SEEDS[:5]:
            for position in POSITIONS[:5]:
                u = sampler.uniform(torch.full((DRAW_ROWS,), seed, dtype=torch.int64),
                                    torch.full((DRAW_ROWS,), position, dtype=torch.int64))
                q, order = sampler._distribution(logits / temperature, None, None, None)
                assert order is None
                draws.append({"temperature": temperature, "seed": seed, "position": position,
                              "tokens": sampler.draw(q, u).tolist()})
    out["draws"] = draws

    out["engine"] = {}
    for name, work in WORKLOADS.items():
        config = make_golden.CONFIGS[name]
        weights = make_golden.tiny_weights(config, make_golden.SEEDS[name])
        prompts = workload_prompts(name)
        with tempfile.TemporaryDirectory() as tmp:
            folder = pathlib.Path(tmp)
            (folder / "config.json").write_text(json.dumps(config))
            save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
            page_bytes = (config["num_hidden_layers"] * 2 * config["num_key_value_heads"] * work["page_size"]
                          * config["head_dim"] * 4)
            runs = {}
            for label, pages, overlap in (("roomy", 64, False), ("tight", -(-work["max_model_len"] // work["page_size"]) + 2, True)):
                engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype=torch.float32,
                                             page_size=work["page_size"], max_seqs=work["max_seqs"],
                                             max_step_tokens=work["max_step_tokens"], max_model_len=work["max_model_len"],
                                             state_memory=page_bytes * (pages + 1), overlap=overlap,
                                             chunk_with_decode=work["chunk_with_decode"], prefix_cache=False), plugins)
                rids = [engine.add(p, SamplingParams(temperature=work["temperature"], seed=s, max_tokens=work["max_tokens"]))
                        for p, s in zip(prompts, work["seeds"])]
                tokens = {rid: [] for rid in rids}
                while engine.has_work():
                    for d in engine.step():
                        tokens[d.rid] += d.token_ids
                stats = engine.stats()
                runs[label] = {"tokens": [tokens[rid] for rid in rids], "preemptions": stats["preemptions"],
                               "mixed_steps": stats["mixed_steps"]}
                engine.close()
            assert runs["roomy"]["tokens"] == runs["tight"]["tokens"], "the reference's own runs disagree"
            out["engine"][name] = {"workload": {k: list(v) if isinstance(v, tuple) else v for k, v in work.items()},
                                   "prompts": prompts, "tokens": runs["roomy"]["tokens"],
                                   "preemptions_tight": runs["tight"]["preemptions"],
                                   "mixed_steps": runs["roomy"]["mixed_steps"],
                                   "checksum": make_golden.checksum(weights)}
    (HERE / "qwen3_tiny_engine.json").write_text(json.dumps(out, indent=1) + "\n")
    print({k: (len(v) if hasattr(v, "__len__") else v) for k, v in out.items()})
    print({n: (e["preemptions_tight"], e["mixed_steps"], e["tokens"][0][:6]) for n, e in out["engine"].items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(pathlib.Path(sys.argv[1]))

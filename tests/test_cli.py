"""The command line (`bin/holon-b200` = `holon_b200.cli.main`): subcommands and options in holon's manner, one flag per
EngineConfig field (core/holon/cli.py:434-456). Generation itself needs the GPU."""
from __future__ import annotations

import dataclasses
import json

import pytest

import plain_qwen3 as plain
from helpers import TINY, make_folder
from holon_b200 import cli
from holon_b200.config.engine import EngineConfig


def test_random_model_and_models(tmp_path, capsys):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY["a"][0]))
    assert cli.main(["random-model", str(config), str(tmp_path / "m"), "--seed", "7"]) == 0
    folder = capsys.readouterr().out.strip()
    stored, weights = plain.read_folder(folder)
    assert stored["hidden_size"] == TINY["a"][0]["hidden_size"] and "model.embed_tokens.weight" in weights
    assert cli.main(["models"]) == 0
    assert "Qwen3ForCausalLM" in capsys.readouterr().out.split()


def test_every_engine_setting_is_a_flag():
    ap_args = ["generate", "some/folder", "--prompt-ids", "1,2", "--dtype", "float32", "--page-size", "32", "--max-seqs", "3",
               "--max-model-len", "100", "--max-step-tokens", "50", "--chunk-with-decode", "8", "--no-cuda-graphs",
               "--no-overlap", "--no-prefix-cache", "--seed", "4", "--n", "2", "--logprobs", "3"]
    seen = {}

    def fake(args):
        seen.update(vars(args))
        return 0
    real, cli.cmd_generate = cli.cmd_generate, fake
    try:
        assert cli.main(ap_args) == 0
    finally:
        cli.cmd_generate = real
    for f in dataclasses.fields(EngineConfig):
        assert f.name in seen, f.name
    config = cli._engine_config(type("A", (), seen))
    assert (config.dtype, config.page_size, config.max_seqs, config.chunk_with_decode) == ("float32", 32, 3, 8)
    assert not config.cuda_graphs and not config.overlap and not config.prefix_cache and config.seed == 4
    assert seen["n"] == 2 and seen["logprobs"] == 3 and seen["prompt_logprobs"] is None


@pytest.mark.gpu
def test_generate_on_the_command_line(tmp_path, capsys):
    folder = make_folder(tmp_path, "b")
    config, weights = plain.read_folder(folder)
    common = ["generate", str(folder), "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6", "--max-tokens", "5", "--dtype",
              "float32", "--max-model-len", "64", "--max-seqs", "4", "--max-step-tokens", "64", "--page-size", "16"]
    assert cli.main(common) == 0
    captured = capsys.readouterr()
    assert "holon-b200: memory: weights" in captured.err and "cache pools" in captured.err   # the account, at the start
    lines = [json.loads(line) for line in captured.out.splitlines()]
    assert [o["prompt_ids"] for o in lines] == [[5, 17, 3], [9, 8, 7, 6]]
    for o in lines:
        assert o["token_ids"] == plain.generate(config, weights, o["prompt_ids"], 5)
    assert cli.main(common + ["--n", "2", "--temperature", "0.8", "--sampling-seed", "3", "--logprobs", "2",
                              "--prompt-logprobs", "0"]) == 0
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines()]
    assert [(o["prompt"], o["index"]) for o in lines] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    for o in lines:
        assert len(o["token_ids"]) == 5 and o["finish_reason"] == "length"
        assert len(o["logprobs"]["token"]) == 5 and all(len(t) == 2 for t in o["logprobs"]["top_ids"])
        assert ("prompt_logprobs" in o) == (o["index"] == 0)
    assert len(lines[0]["prompt_logprobs"]["token"]) == 2 and lines[0]["token_ids"] != lines[1]["token_ids"]


def test_generate_streams_sequences_and_logprobs_with_the_plain_kernel_table(tmp_path, capsys, monkeypatch):
    """The command's two ways of generating (whole prompts; `add` / `step` for --n and log-probabilities) on the CPU,
    the engine built with the plain torch kernel table in place of the CUDA kernels."""
    import holon_b200.engine as engine_module
    from ref_kernels import RefKernels

    class CpuEngine(engine_module.Engine):
        def __init__(self, config):
            config.device, config.state_memory = "cpu", 1 << 20
            super().__init__(config, kernels=RefKernels())
    monkeypatch.setattr(engine_module, "Engine", CpuEngine)
    folder = make_folder(tmp_path, "b")
    config, weights = plain.read_folder(folder)
    common = ["generate", str(folder), "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6", "--max-tokens", "5", "--dtype",
              "float32", "--max-model-len", "64", "--max-seqs", "4", "--max-step-tokens", "64", "--page-size", "16"]
    assert cli.main(common) == 0
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines()]
    assert [o["token_ids"] for o in lines] == [plain.generate(config, weights, p, 5) for p in ([5, 17, 3], [9, 8, 7, 6])]
    assert cli.main(common + ["--n", "2", "--temperature", "0.8", "--sampling-seed", "3", "--logprobs", "2",
                              "--prompt-logprobs", "0"]) == 0
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines()]
    assert [(o["prompt"], o["index"]) for o in lines] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert lines[0]["token_ids"] == plain.generate(config, weights, [5, 17, 3], 5, 0.8, 3)
    assert all(len(o["logprobs"]["token"]) == 5 and ("prompt_logprobs" in o) == (o["index"] == 0) for o in lines)

"""The checks must be able to fail. Each test plants one bug of the kind the replay tests exist to catch and asserts
that the very comparison those tests use (`replay_tools.compare`) rejects the result, in true 32-bit and in bfloat16;
the unplanted run passes the same comparison. The reference's judge proves its own checks the same way, with
deliberately broken engines (judge/holon_judge/planted.py:1-30).

Planted: a rotation base 1 % off; a norm eps ten times too large; a block-table entry one page off; a cache write one
place off; a causal mask off by one (a query that cannot see itself; a query that sees one key ahead); the query head
to KV head mapping `h % kv_heads` in place of `h // group`. The engine runs on the CPU with the plain kernel table
(`ref_kernels.RefKernels`), whose functions are overridden one at a time; the bugs that sit in the configuration run
on the GPU kernels too (`-m gpu`), and one bug is planted in front of the CUDA attention kernel.

Two of the bugs hide under bfloat16's rounding at the tiny models' usual weights and lengths, so the inputs are made
to show them: a 1 % error of the rotation base turns the pairs by a share of the position, which a request of 1,200
tokens makes larger than the rounding (over the 133 tokens of the other requests it is not); and eps matters only
beside a small mean square, so the embedding table is scaled by a tenth (the residual stream's mean square then is of
the size of eps).
"""
from __future__ import annotations

import json
import shutil

import pytest
import torch

import plain_qwen3 as plain
from helpers import make_folder, random_prompt
from holon_b200.replay import Replayer
from ref_kernels import RefKernels
from replay_tools import compare, exact_and_rounded, mixed_trace, portions, run

LENGTHS = (70, 133, 37, 96)


class OtherPage(RefKernels):
    """Reads the second logical page of every request from the physical page after the right one."""

    def paged_attention(self, out, q, kv, block_table, rows, scale, window):
        table = block_table.clone()
        table[:, 1] = (table[:, 1] + 1) % (kv.shape[0] - 1)
        super().paged_attention(out, q, kv, table, rows, scale, window)


class LateWrite(RefKernels):
    """Writes every key and value one place later than its position."""

    def qk_norm_rope_kv_write(self, q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                              write_index, heads, kv_heads, head_dim):
        if write_index is not None:
            places = (kv.shape[0] - 1) * kv.shape[3]
            write_index = torch.where(write_index >= 0, (write_index + 1) % places, write_index)
        super().qk_norm_rope_kv_write(q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                                      write_index, heads, kv_heads, head_dim)


class Masked(RefKernels):
    """The causal mask off by one: `shift` -1 hides a query's own key, +1 shows the key after it."""

    def __init__(self, shift):
        self.shift = shift

    def paged_attention(self, out, q, kv, block_table, rows, scale, window):
        page_size, hq, hkv = kv.shape[3], q.shape[1], kv.shape[2]
        out.zero_()
        qs, slots, lens = rows.query_start.tolist(), rows.row_slot.tolist(), rows.kv_len.tolist()
        for b in range(rows.n_rows):
            s, e, n = qs[b], qs[b + 1], lens[b]
            pages = block_table[slots[b], : -(-n // page_size)].long()
            k, v = (kv[pages, i].transpose(1, 2).reshape(-1, hkv, kv.shape[4])[:n].float()
                    .repeat_interleave(hq // hkv, dim=1) for i in (0, 1))
            scores = torch.einsum("qhd,khd->hqk", q[s:e].float(), k) * scale
            pos = torch.arange(n - (e - s), n)[:, None]
            hidden = torch.arange(n)[None, :] > pos + self.shift
            hidden[:, 0] = False                                      # (never a row without any key: no NaN to give it away)
            probs = scores.masked_fill(hidden, float("-inf")).softmax(-1)
            out[s:e] = torch.einsum("hqk,khd->qhd", probs, v).to(out.dtype)


class WrongGroup(RefKernels):
    """Query head h reads KV head h % kv_heads instead of h // (heads / kv_heads)."""

    def paged_attention(self, out, q, kv, block_table, rows, scale, window):
        hq, hkv = q.shape[1], kv.shape[2]
        order = torch.tensor([(h % hkv) * (hq // hkv) + h // hkv for h in range(hq)])   # a permutation of the query heads
        swapped = torch.empty_like(out)
        super().paged_attention(swapped, q[:, order].contiguous(), kv, block_table, rows, scale, window)
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(hq)
        out.copy_(swapped[:, inverse])


def altered_folder(tmp_path, folder, label, **changes):
    """A copy of `folder` whose config.json differs in `changes` (the weights stay)."""
    copy = tmp_path / f"{folder.name}_{label}"
    shutil.copytree(folder, copy)
    config = json.loads((copy / "config.json").read_text())
    config.update({k: config[k] * v for k, v in changes.items()})
    (copy / "config.json").write_text(json.dumps(config))
    return copy


@pytest.fixture(scope="module", params=["a", "b"])
def model(request, tmp_path_factory):
    from safetensors.torch import load_file, save_file
    tmp = tmp_path_factory.mktemp("planted")
    folder = make_folder(tmp, request.param)
    tensors = load_file(str(folder / "model.safetensors"))
    table = tensors["model.embed_tokens.weight"]
    tensors["model.embed_tokens.weight"] = (table.float() * 0.1).to(table.dtype)      # a small stream: eps counts
    save_file(tensors, str(folder / "model.safetensors"))
    config, weights = plain.read_folder(folder)
    prompts = {f"r{i}": random_prompt(config["vocab_size"], n, 40 + i) for i, n in enumerate(LENGTHS)}
    prompts["long"] = random_prompt(config["vocab_size"], 1200, 9)
    want = {rid: exact_and_rounded(config, weights, ids) for rid, ids in prompts.items()}
    return request.param, tmp, folder, prompts, want


def replay(folder, dtype, prompts, kernels=None, device="cpu"):
    """Four requests mixed in a small pool (see replay_tools.mixed_trace), pages of 16."""
    r = Replayer(str(folder), dtype, max_tokens=448, device=device, kernels=kernels, page_size=16)
    return run(r, mixed_trace(prompts))


def replay_long(folder, dtype, prompts, kernels=None, device="cpu"):
    """One request of 1,200 tokens in four portions."""
    r = Replayer(str(folder), dtype, max_tokens=1216, device=device, kernels=kernels, page_size=16)
    parts = portions(prompts["long"], [600, 2, 300, 298])
    return run(r, [([("long", part)], ["long"] if i == len(parts) - 1 else []) for i, part in enumerate(parts)])


def rejected(got, want, dtype) -> bool:
    try:
        compare(got, want, dtype)
    except AssertionError:
        return True
    return False


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_planted_bug_is_rejected(model, dtype):
    name, tmp, folder, prompts, want = model
    compare(replay(folder, dtype, prompts, RefKernels()), want, dtype)           # unplanted: accepted
    compare(replay_long(folder, dtype, prompts, RefKernels()), want, dtype)
    theta = altered_folder(tmp, folder, f"theta_{dtype}", rope_theta=1.01)
    assert rejected(replay_long(theta, dtype, prompts, RefKernels()), want, dtype), "a rotation base 1 % off was accepted"
    planted = {
        "eps ten times too large": (altered_folder(tmp, folder, f"eps_{dtype}", rms_norm_eps=10.0), RefKernels()),
        "a block-table entry one page off": (folder, OtherPage()),
        "a cache write one place off": (folder, LateWrite()),
        "a query that cannot see itself": (folder, Masked(-1)),
        "a query that sees one key ahead": (folder, Masked(+1)),
    }
    if name == "a":                       # (with one KV head, as in configuration b, both mappings are the same)
        planted["query heads mapped to the wrong KV head"] = (folder, WrongGroup())
    missed = [bug for bug, (where, kernels) in planted.items()
              if not rejected(replay(where, dtype, prompts, kernels), want, dtype)]
    assert not missed, f"{dtype}: the comparison accepted {missed}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_planted_bugs_are_rejected_on_the_gpu(model, dtype):
    """Through the CUDA kernels: the two bugs that sit in the configuration, and a block-table entry one page off
    planted in front of the attention kernel (the kernel table is wrapped for the one call)."""
    from holon_b200.kernels import load_kernels
    name, tmp, folder, prompts, want = model
    real = load_kernels("cuda:0")

    class OtherPageOnTheGpu:
        def __getattr__(self, attribute):
            return getattr(real, attribute)

        def paged_attention(self, out, q, kv, block_table, rows, scale, window):
            table = block_table.clone()
            table[:, 1] = (table[:, 1] + 1) % (kv.shape[0] - 1)
            real.paged_attention(out, q, kv, table, rows, scale, window)

    compare(replay(folder, dtype, prompts, device="cuda:0"), want, dtype)
    compare(replay_long(folder, dtype, prompts, device="cuda:0"), want, dtype)
    theta = altered_folder(tmp, folder, f"gpu_theta_{dtype}", rope_theta=1.01)
    assert rejected(replay_long(theta, dtype, prompts, device="cuda:0"), want, dtype), "a rotation base 1 % off was accepted"
    planted = {
        "eps ten times too large": (altered_folder(tmp, folder, f"gpu_eps_{dtype}", rms_norm_eps=10.0), None),
        "a block-table entry one page off": (folder, OtherPageOnTheGpu()),
    }
    missed = [bug for bug, (where, kernels) in planted.items()
              if not rejected(replay(where, dtype, prompts, kernels, device="cuda:0"), want, dtype)]
    assert not missed, f"{dtype}: the comparison accepted {missed}"

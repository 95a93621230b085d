"""A part that brings CUDA of its own: a toy feed-forward whose activation is a kernel in `tests/toy_kernels/`,
compiled into a library beside the engine's through the kernel table's extension seam. The part is defined,
registered, built and stepped from this file alone; the framework's kernel table, its C header and its library stay as
they are. The model that holds it is compared with the formulas written out; a call the kernel refuses raises the
table's error with the kernel's own text; and a bounded wait inside the part's kernel that runs out reaches the
engine's status word like a wait of the engine's own kernels."""
from __future__ import annotations

import pathlib

import pytest
import torch

import plain_qwen3 as plain
from holon_b200.config import LayerSpec, ModelSpec, PartRef, Run, WeightRule, register_architecture, unregister_architecture
from holon_b200.engine import StepEntry, build
from holon_b200.kernels.cuda import KernelError
from holon_b200.parts import Part, register_part, unregister_part
from holon_b200.weights import RandomSource
from test_gpu_toy_parts import EPS, HEAD_DIM, HEADS, KV_HEADS, plain_attention

pytestmark = pytest.mark.gpu
SOURCES = [pathlib.Path(__file__).resolve().parent / "toy_kernels" / "toy_gate.cu"]
BUILD_DIR = None                                       # set by the fixture: a temporary folder


class GatedProduct(Part):
    """out = W · (x ⊙ sigmoid(scale ⊙ x)): the activation in the part's own kernel, the product in the table's."""

    def __init__(self, ctx, *, hidden, layer=0):
        super().__init__()
        self.ctx, self.hidden = ctx, hidden
        self.scale = self.add_param("scale", (hidden,), "gain")
        self.weight = self.add_param("weight", (hidden, hidden), "matrix")

    def finalize(self):
        """(The constructor only declares: a model is also built without a device, to list its parameters.)"""
        self.ext = self.ctx.kernels.extension("toy_gate", SOURCES, build_dir=BUILD_DIR, status_mirrors=("toy_status_mirror",))
        self.scale32 = self.scale.tensor.float().contiguous()

    def forward(self, x, step):
        ext = self.ext
        ext.check(x, self.scale32)
        gated, out = torch.empty_like(x), torch.empty_like(x)
        ext.call("toy_gate", ext.ptr(gated), ext.ptr(x), int(x.dtype == torch.bfloat16), ext.ptr(self.scale32),
                 x.shape[0], x.shape[1])
        self.ctx.kernels.linear(out, gated, self.weight.tensor)
        return out


def gate_recipe(c):
    norm = PartRef.of("norm", "rmsnorm", eps=EPS)
    attention = PartRef.of("mixer", "gqa", heads=HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, qk_norm=norm, window=0,
                           position=PartRef.of("position", "rope", theta=1e4, rotary_dim=HEAD_DIM))
    layer = LayerSpec(PartRef.of("block", "prenorm"), attention, PartRef.of("ffn", "toy_gated_product"), norm)
    return ModelSpec(hidden=c["hidden"], vocab=c["vocab"], layers=(layer, layer), order=(Run(0, 0), Run(1, 1)),
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=True),
                     weight_rules=(WeightRule("{rest}", "{rest}"),))


def plain_forward(model, ids):
    f = lambda p: p.tensor.float().cpu()
    h = plain.embedding(ids, f(model.embed.weight))
    for block in model.layers:
        h = h + plain_attention(plain.rms_norm(h, f(block.input_norm.weight), EPS), block.mixer)
        x = plain.rms_norm(h, f(block.post_norm.weight), EPS)
        h = h + (x * torch.sigmoid(f(block.ffn.scale) * x)) @ f(block.ffn.weight).T
    return plain.rms_norm(h, f(model.norm.weight), EPS) @ f(model.embed.weight).T


@pytest.fixture()
def registered(tmp_path_factory):
    global BUILD_DIR
    BUILD_DIR = tmp_path_factory.mktemp("toy_build")
    register_part("ffn", "toy_gated_product", GatedProduct)
    register_architecture("ToyGatedForCausalLM", dict, gate_recipe)
    yield
    unregister_part("ffn", "toy_gated_product")
    unregister_architecture("ToyGatedForCausalLM")


def built(dtype="float32"):
    config = {"architectures": ["ToyGatedForCausalLM"], "hidden": 72, "vocab": 131}
    return build(RandomSource(config, seed=5, dtype=torch.float32), dtype=dtype, device="cuda:0", page_size=8,
                 max_seqs=2, max_model_len=64, max_step_tokens=64, pages=10)


def test_a_part_with_a_kernel_of_its_own(registered):
    b = built()
    ext = b.model.layers[0].ffn.ext
    assert ext is b.model.layers[1].ffn.ext and ext.path.parent == BUILD_DIR      # compiled once, where it was told to
    assert ext.path != b.ctx.kernels.path and ext.path.name.startswith("libholon_b200x_toy_gate_")
    ids = torch.randint(0, 131, (41,), generator=torch.Generator().manual_seed(2)).tolist()
    want = plain_forward(b.model, ids)
    for portions in ([41], [30] + [1] * 11, [2, 17, 3, 19]):
        slot, at, rows = b.cache.admit(), 0, []
        for n in portions:
            b.cache.reserve(slot, at + n)
            rows.append(b.runner.step([StepEntry(slot, ids[at:at + n], at, range(n))]))
            at += n
        b.cache.release(slot)
        got = torch.cat(rows).cpu()
        assert (got - want).abs().max() < 1e-4, (portions, float((got - want).abs().max()))
        assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_an_extensions_refusal_and_missing_function(registered):
    b = built()
    ext = b.model.layers[0].ffn.ext
    x = torch.zeros(2, 72, device="cuda:0")
    with pytest.raises(KernelError, match="toy_gate: dtype 7"):
        ext.call("toy_gate", ext.ptr(x), ext.ptr(x), 7, ext.ptr(x), 2, 72)
    with pytest.raises(KernelError, match="no such function"):
        ext.call("toy_other")
    with pytest.raises(KernelError, match="contiguous"):
        ext.check(x.t())


def test_a_wait_in_a_parts_own_kernel_reaches_the_status_word(registered):
    b = built()
    kernels, ext = b.ctx.kernels, b.model.layers[0].ffn.ext
    torch.cuda.synchronize()
    kernels.clear_status()
    ext.call("toy_wait_that_runs_out", 200)
    torch.cuda.synchronize()
    assert kernels.status() == (14 << 28) | 1
    kernels.clear_status()
    assert kernels.status() == 0

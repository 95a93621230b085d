"""The kernel table of the product path: hand-written CUDA for sm_100a, called through the library's C interface.

Every method takes torch tensors on one CUDA device, checks what the kernel assumes (device, dtype, contiguity,
shapes) and enqueues the kernel on torch's current stream. There is no other path: a size a kernel refuses raises
`KernelError` with the kernel's own message. Plain bfloat16 matrix products of more than 16 rows go to cuBLAS through
torch, as the reference's go through `torch.nn.functional.linear` (std/holon_std/ops/units.py:223-229); products
of up to 16 rows, SwiGLU's product with its activation, and float32 products run the library's own kernels.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .build import extension_path, library_path

_CODES = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {t.dtype}") from None


class _ChainPhase(ctypes.Structure):
    """hb_chain_phase of csrc/api.h."""

    _fields_ = [(name, ctypes.c_void_p) for name in ("w", "x", "out", "h", "next_weight", "ss_out", "ss_in")] \
        + [(name, ctypes.c_int) for name in ("n", "k", "mode", "inter", "out_f32", "next_weight_f32", "parts_in", "dim_in")] \
        + [("next_offset", ctypes.c_float), ("eps_in", ctypes.c_float)]


class Extension:
    """The functions of a part's own CUDA library (`CudaKernels.extension`). `ext.call("fn", a, b, ...)` runs
    `int fn(a, b, ..., stream)` on torch's current stream after whatever the table still has queued, and raises
    `KernelError` with the library's text when it returns non-zero. `ptr`, `i32` and `check` are the table's own
    helpers for arguments: a tensor's address (0 for None), the same with the dtype checked, and device and contiguity."""

    def __init__(self, kernels: "CudaKernels", name: str, path, status_mirrors=()) -> None:
        self.kernels, self.name, self.path = kernels, name, path
        self.lib = ctypes.CDLL(str(path))
        self._fn: dict = {}
        self.ptr, self.i32, self.check = kernels._p, kernels._i32, kernels._check
        for fn in status_mirrors:             # its bounded waits report into the word that the engine reads
            word = ctypes.POINTER(ctypes.c_uint)()
            with torch.cuda.device(kernels.device):
                if kernels.lib.hb_status_word_device(ctypes.byref(word)) or getattr(self.lib, fn)(word):
                    raise KernelError(f"{name}.{fn}: {kernels.lib.hb_last_error().decode()}")

    def call(self, fn: str, *args) -> None:
        self.kernels._call_in(self.lib, self._fn, fn, *args)


class CudaKernels:
    name = "cuda sm_100a"

    def __init__(self, device) -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(f"the engine runs on a CUDA device; {self.device} is none")
        self.path = library_path()
        self.lib = ctypes.CDLL(str(self.path), mode=ctypes.RTLD_GLOBAL)      # (extensions use its hb_set_error)
        self._extensions: dict[str, Extension] = {}
        self.lib.hb_last_error.restype = ctypes.c_char_p
        self._fn = {}
        self._index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        self.launches = 0
        self._splits: dict = {}
        # Which kernel attends for rows of several tokens: "tcgen05" (csrc/attention_tcgen05.cu, for head size 128 and
        # pages of a multiple of 64 tokens; every other shape takes the mma.sync kernel) or "mma" (mma.sync always:
        # any head size up to 256 in steps of 16, any page size).
        self.prefill_attention = os.environ.get("HOLON_B200_PREFILL_ATTENTION", "tcgen05")
        if self.prefill_attention not in ("mma", "tcgen05"):
            raise KernelError(f"HOLON_B200_PREFILL_ATTENTION must be mma or tcgen05, not {self.prefill_attention!r}")
        # Which kernel multiplies bfloat16 matrices of more than SKINNY_ROWS rows: "auto" (the default: the library
        # through torch, as the reference uses one there, except SwiGLU's gate/up product, which goes to the
        # hand-written tcgen05 kernel with the activation in its epilogue where that is faster than the library's
        # product plus an activation kernel), "cublas" (the library always) or "tcgen05" (csrc/gemm_tcgen05*.cu always).
        self.gemm = os.environ.get("HOLON_B200_GEMM", "auto")
        if self.gemm not in ("auto", "cublas", "tcgen05"):
            raise KernelError(f"HOLON_B200_GEMM must be auto, cublas or tcgen05, not {self.gemm!r}")
        self.gemm_pair = os.environ.get("HOLON_B200_GEMM_PAIR", "1") != "0"   # the tcgen05 product by CTA pairs
        self.attention_bf16 = "fast"          # "generic" forces the CUDA-core kernel for bfloat16 too (tests)
        # How the keys of rows that bring one token are shared out when one CTA per (row, kv head) is too few:
        # "splits" (every row cut into the same number of parts), "balanced" (every CTA of one GPU-filling wave takes
        # the same number of 64-key tiles, whatever the rows' lengths) or "auto" (balanced for a batch with one row far
        # longer than the others, where equal cuts leave most CTAs with almost nothing; see decode_mode).
        self.decode_attention = os.environ.get("HOLON_B200_DECODE_ATTENTION", "auto")
        if self.decode_attention not in ("auto", "balanced", "splits"):
            raise KernelError(f"HOLON_B200_DECODE_ATTENTION must be auto, balanced or splits, not {self.decode_attention!r}")
        self.decode_cluster = os.environ.get("HOLON_B200_DECODE_CLUSTER", "1") != "0"   # splits of up to 16 merge in the kernel
        self.fused_qkv = os.environ.get("HOLON_B200_FUSED_QKV", "1") != "0"   # decode steps: norm, rotation, cache write in the product
        self.fused_norm = os.environ.get("HOLON_B200_FUSED_NORM", "1") != "0"   # decode steps: residual sum and next norm in the product before
        # Where csrc/gemm_mid.cu (tcgen05, the k range split over a thread-block cluster) runs (HOLON_B200_MID). "auto", the
        # default, for weights of 32 MB or more: SwiGLU's product at up to MID_ROWS rows (one CTA a tile, no sum over a
        # cluster; its idle warps add up the row scales while the weights stream, which costs the mma.sync kernel a trip
        # to the L2 at the end of every CTA: back to back in a graph on rows that lack their norm's scale, Qwen3-8B
        # sizes, 36.3 us against 38.0 at 8 rows, 36.3 against 37.4 at 1, 36.5 against 42.3 at 16; from 17 rows level
        # with the library's product, and the activation kernel is saved), and the attention's first product at 9 to
        # 16 rows (14.4 us against 15.1 at 16 rows: the mma.sync kernel reads x for a second tile of eight rows there;
        # at 8 rows it is 13.9 against 14.1 the other way). o_proj and down stay with the mma.sync kernel up to 16 rows
        # (8.5 and 18.6 us against 10.3 and 20.6: a launch of this kernel costs 5 us before its first byte counts, the
        # other 2). "all": steps of 17 to MID_ROWS rows keep every fused product there, instead of the library's
        # product and kernels of their own for the work around it; "swiglu": of those only SwiGLU's, whatever the
        # weight's size. Measured, decode steps of 64 / 32 / 17 rows at 2,304 keys: 7.31 / 5.25 / 4.46 ms with the library
        # alone, 7.24 / 5.24 / 4.45 with SwiGLU's product here, 7.48 / 5.28 / 4.48 with "all" (a clustered product costs
        # 3 us more than the library's, which is what the kernels it saves cost). "0": never. `mid_split`: tests force
        # the cluster size (0: chosen per launch).
        self.mid_mode = os.environ.get("HOLON_B200_MID", "auto")
        if self.mid_mode not in ("0", "auto", "swiglu", "all"):
            raise KernelError(f"HOLON_B200_MID must be 0, auto, swiglu or all, not {self.mid_mode!r}")
        self.mid_split = 0
        self.mid_launches = 0
        self.mid_min_rows = int(os.environ.get("HOLON_B200_MID_MIN_ROWS", "9"))   # the attention's first product: fewer rows stay with the mma.sync kernel
        # Steps of 17 to WIDE_ROWS rows and weights below MID_WEIGHT elements (small models, where a kernel is its launch):
        # the mma.sync kernel with four tiles of x a warp keeps the fused epilogues ("1"), or the library multiplies and
        # kernels of their own do the rest ("0").
        self.skinny32 = os.environ.get("HOLON_B200_SKINNY32", "1") != "0"
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.decode_ctas = None               # tests: a fixed number of CTAs for the balanced kernel
        self.prefill_tile = None              # tests, microbench: 128 or 256 queries a CTA of the tcgen05 prefill kernel
        # Decode steps: the products of a layer that follow one another on the same few rows (the mixer's last, the
        # feed-forward's two, the next mixer's first) can be queued and run in one launch; every other call of this table
        # runs what is queued first. HOLON_B200_CHAIN: "tickets" (csrc/gemm_tickets.cu: every CTA a tile of one of the
        # products, drawn in order, so that a product starts while the one before ends), "ring" (csrc/gemm_chain.cu: one
        # persistent kernel with a shared-memory ring; slower as measured) or "0" (every product its own launch).
        self.chain = {"0": "", "1": "tickets"}.get(os.environ.get("HOLON_B200_CHAIN", "0"), os.environ.get("HOLON_B200_CHAIN", "0"))
        if self.chain not in ("", "tickets", "ring"):
            raise KernelError(f"HOLON_B200_CHAIN must be 0, tickets or ring, not {self.chain!r}")
        self.chain_cooperative = os.environ.get("HOLON_B200_CHAIN_COOPERATIVE", "1") != "0"
        self._pending: list = []              # (phase, tensors it names) of products queued, in order
        self.chain_launches = self.chain_phases = 0
        self.lib.hb_gemm_chain_capacity.restype = ctypes.c_int
        with torch.cuda.device(self.device):
            self._chain_slots = int(self.lib.hb_gemm_chain_capacity())
        if self._chain_slots < 1:
            raise KernelError("hb_gemm_chain_capacity: the device runs no CTA of the chained products' kernel")
        self._chain_sync = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._chain_flags = torch.zeros(self._chain_slots, dtype=torch.int32, device=self.device)
        self._chain_scratch = torch.empty(self._chain_slots * 512, dtype=torch.float32, device=self.device)
        self._ticket_state = torch.zeros(8, dtype=torch.int32, device=self.device)
        # One word of page-locked host memory that a kernel's bounded wait writes when it gives up (csrc/status.cu)
        word = ctypes.POINTER(ctypes.c_uint)()
        with torch.cuda.device(self.device):
            if self.lib.hb_status_word(ctypes.byref(word)):
                raise KernelError(f"hb_status_word: {self.lib.hb_last_error().decode()}")
        self._status_word = word

    # ------------------------------------------------------------------ plumbing
    @property
    def mid(self) -> bool:
        """Whether steps of 17 to MID_ROWS rows keep their fused products (csrc/gemm_mid.cu)."""
        return self.mid_mode == "all"

    WIDE_ROWS = 32                            # rows the mma.sync kernel takes with four tiles of x a warp

    def _wide_takes(self, m: int, weight, stride: int | None = None) -> bool:
        """Whether a product of 17 to WIDE_ROWS rows with a small `weight` runs in the 32-row mma.sync kernel (`stride`:
        the tokens a part of its rows' partial sums holds, if the rows are parts.base.Scaled: that kernel reads 32)."""
        return self.skinny32 and self.SKINNY_ROWS < m <= self.WIDE_ROWS and weight.numel() < self.MID_WEIGHT \
            and stride in (None, self.WIDE_ROWS) and not (self.mid_mode == "all" and stride is None)

    MID_WEIGHT = 16 << 20                     # elements of a weight from which "auto" sends a product to csrc/gemm_mid.cu

    def _mid_takes(self, m: int, weight, mode: int) -> bool:
        """Whether the product of `m` rows with `weight` and the epilogue `mode` (1 SwiGLU, 2 q/k norm, rotation and
        cache write) runs in csrc/gemm_mid.cu rather than in the kernel for up to SKINNY_ROWS rows."""
        if self.mid_mode == "0" or m > self.MID_ROWS or (self.chain and m <= self.SKINNY_ROWS):
            return False                                   # (chained products are the mma.sync kernel's tiles)
        large = weight.numel() >= self.MID_WEIGHT
        if m <= self.SKINNY_ROWS:                          # SwiGLU's at any number of rows, the attention's first from 9 on
            return large and (mode == 1 or (mode == 2 and m >= self.mid_min_rows))
        return self.mid_mode == "all" or (mode == 1 and (self.mid_mode == "swiglu" or (large and self.gemm != "cublas")))

    def _call(self, name: str, *args) -> None:
        if self._pending:                      # what is queued comes first: this call may read what it writes
            self.flush()
        self._launch(name, *args)

    def _launch(self, name: str, *args) -> None:
        fn = self._fn.get(name)
        if fn is None:
            fn = self._fn[name] = getattr(self.lib, name)
            fn.restype = ctypes.c_int
        code = fn(*args, ctypes.c_void_p(self._stream()))
        self.launches += 1
        if code:
            raise KernelError(f"{name}: {self.lib.hb_last_error().decode()}")

    def _call_in(self, lib, cache: dict, name: str, *args) -> None:
        """`_call` for a function of another library (an extension's)."""
        if self._pending:
            self.flush()
        fn = cache.get(name)
        if fn is None:
            try:
                fn = cache[name] = getattr(lib, name)
            except AttributeError:
                raise KernelError(f"{name}: the extension's library exports no such function") from None
            fn.restype = ctypes.c_int
        code = fn(*args, ctypes.c_void_p(self._stream()))
        self.launches += 1
        if code:
            raise KernelError(f"{name}: {self.lib.hb_last_error().decode() or f'returned {code}'}")

    def extension(self, name: str, sources, build_dir=None, status_mirrors=()) -> Extension:
        """A part's own CUDA files as a library beside this one: compiled on first use (kernels/build.py:
        `extension_path`), loaded once per table. The part calls its functions through the `Extension` it gets; this
        file, api.h and the main library stay as they are. `status_mirrors`: the names its files gave to
        HB_DEFINE_STATUS_MIRROR (csrc/tcgen05.cuh), one per file with bounded waits; `status()` then shows a wait of
        theirs that gave up, and the engine stops on it as on any other."""
        ext = self._extensions.get(name)
        if ext is None:
            path = extension_path(name, sources, build_dir)
            ext = self._extensions[name] = Extension(self, name, path, status_mirrors)
        return ext

    # ---- products queued for one persistent kernel (decode steps)
    MAX_CHAIN = 8                              # phases a launch takes (csrc/gemm_chain.cu)
    MAX_TICKETS = 4                            # products a launch takes (csrc/gemm_tickets.cu)

    def _queue(self, *, w, x, out, mode: int, n: int, inter: int = 0, h=None, next_weight=None, next_offset: float = 0.0,
               ss_out=None, scaled=None) -> None:
        if len(self._pending) >= (self.MAX_CHAIN if self.chain == "ring" else self.MAX_TICKETS):
            self.flush()
        y = scaled.y if scaled is not None else x
        phase = _ChainPhase(w=w.data_ptr(), x=y.data_ptr(), out=out.data_ptr(), h=h.data_ptr() if h is not None else None,
                            next_weight=next_weight.data_ptr() if next_weight is not None else None,
                            ss_out=ss_out.data_ptr() if ss_out is not None else None,
                            ss_in=scaled.ss.data_ptr() if scaled is not None else None, n=n, k=y.shape[1], mode=mode,
                            inter=inter, out_f32=int(out.dtype == torch.float32),
                            next_weight_f32=int(next_weight is not None and next_weight.dtype == torch.float32),
                            parts_in=scaled.ss.shape[0] if scaled is not None else 0,
                            dim_in=scaled.dim if scaled is not None else 0, next_offset=float(next_offset),
                            eps_in=float(scaled.eps) if scaled is not None else 0.0)
        keep = (w, x, out, h, next_weight, ss_out, scaled)            # (the tensors stay alive until the launch)
        if self._pending and self._pending[0][2] != y.shape[0]:
            self.flush()
        self._pending.append((phase, keep, y.shape[0]))

    def flush(self) -> None:
        """Launches what is queued: one persistent kernel for all of it. Everything this table's other calls do comes
        after it; whoever reads a queued product's output by other means (torch operations) calls this first."""
        if not self._pending:
            return
        pending, self._pending = self._pending, []
        phases = (_ChainPhase * len(pending))(*[p for p, _, _ in pending])
        if self.chain == "ring":
            self._launch("hb_gemm_chain", phases, len(pending), pending[0][2], self._p(self._chain_sync),
                         self._p(self._chain_scratch), self._p(self._chain_flags), self._chain_slots, int(self.chain_cooperative))
        else:
            self._launch("hb_gemm_tickets", phases, len(pending), pending[0][2], self._p(self._ticket_state))
        self.chain_launches += 1
        self.chain_phases += len(pending)

    def _chains(self, m: int, k: int, *tensors) -> bool:
        """Whether a product of `m` rows over `k` columns of these bfloat16 tensors may be queued."""
        return bool(self.chain) and 0 < m <= self.SKINNY_ROWS and k % 8 == 0 \
            and all(t.dtype == torch.bfloat16 and t.data_ptr() % 16 == 0 for t in tensors)

    def _stream(self) -> int:
        """The handle of torch's current stream on the device (a few hundred kernels a step ask for it)."""
        if self._raw_stream is not None:
            return self._raw_stream(self._index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, *tensors: torch.Tensor | None) -> None:
        index = self._index
        for t in tensors:
            if t is None or (t.is_cuda and t.get_device() == index and t.is_contiguous()):
                continue
            if t.device != self.device:
                raise KernelError(f"a tensor lives on {t.device}, the kernels run on {self.device}")
            raise KernelError(f"kernels take contiguous tensors; got strides {t.stride()} for shape {tuple(t.shape)}")

    @staticmethod
    def _p(t: torch.Tensor | None) -> ctypes.c_void_p:
        return ctypes.c_void_p(t.data_ptr() if t is not None else 0)

    @staticmethod
    def _i32(t: torch.Tensor | None, what: str) -> ctypes.c_void_p:
        if t is not None and t.dtype != torch.int32:
            raise KernelError(f"{what} must be int32, not {t.dtype}")
        return ctypes.c_void_p(t.data_ptr() if t is not None else 0)

    # ------------------------------------------------------------------ kernels
    def embed(self, out, table, ids) -> None:
        self._check(out, table, ids)
        if out.dtype != torch.float32 or out.shape != (ids.shape[0], table.shape[1]):
            raise KernelError("embed: out must be float32 [tokens, hidden]")
        self._call("hb_embed", self._p(out), self._p(table), _code(table), self._i32(ids, "ids"),
                   ids.shape[0], table.shape[1], table.shape[0])

    def rmsnorm(self, out, x, weight, eps, offset) -> None:
        self._check(out, x, weight)
        if out.shape != x.shape or weight.shape != (x.shape[-1],):
            raise KernelError("rmsnorm: out and x must have one shape, weight [dim]")
        rows = x.numel() // x.shape[-1]
        self._call("hb_add_rmsnorm", self._p(out), _code(out), self._p(x), _code(x), self._p(None), self._p(weight),
                   _code(weight), ctypes.c_float(eps), ctypes.c_float(offset), self._p(None), rows, x.shape[-1])

    def add_rmsnorm(self, out, h, delta, weight, eps, offset, index) -> None:
        self._check(out, h, delta, weight, index)
        rows = index.shape[0] if index is not None else h.shape[0]
        if h.dtype != torch.float32 or out.shape != (rows, h.shape[1]) or weight.shape != (h.shape[1],):
            raise KernelError("add_rmsnorm: h must be float32 [tokens, dim], out [rows, dim], weight [dim]")
        if delta is not None and (delta.shape != h.shape or delta.dtype != out.dtype):
            raise KernelError("add_rmsnorm: delta must have h's shape and out's dtype")
        self._call("hb_add_rmsnorm", self._p(out), _code(out), self._p(h), 0, self._p(delta), self._p(weight),
                   _code(weight), ctypes.c_float(eps), ctypes.c_float(offset), self._i32(index, "index"), rows,
                   h.shape[1])

    def silu_mul(self, out, gate_up) -> None:
        self._check(out, gate_up)
        if gate_up.shape != (out.shape[0], 2 * out.shape[1]) or out.dtype != gate_up.dtype:
            raise KernelError("silu_mul: gate_up must be [tokens, 2 * inter] of out's dtype")
        self._call("hb_silu_mul", self._p(out), self._p(gate_up), _code(out), out.shape[0], out.shape[1])

    def qk_norm_rope_kv_write(self, q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                              write_index, heads, kv_heads, head_dim) -> None:
        self._check(q_out, qkv, positions, table, q_weight, k_weight, kv, write_index)
        t = qkv.shape[0]
        if qkv.shape != (t, (heads + 2 * kv_heads) * head_dim) or q_out.shape != (t, heads, head_dim) \
                or q_out.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv_write: qkv must be [tokens, (heads + 2 kv_heads) head_dim], q_out "
                              "[tokens, heads, head_dim], of one dtype")
        if table is not None and (table.dtype != torch.float32 or table.shape[1] != rotary_dim):
            raise KernelError("qk_norm_rope_kv_write: the rotation table must be float32 [positions, rotary_dim]")
        if kv is not None and (kv.dtype != qkv.dtype or kv.shape[1:3] != (2, kv_heads) or kv.shape[4] != head_dim):
            raise KernelError("qk_norm_rope_kv_write: kv must be [pages, 2, kv_heads, page_size, head_dim] of qkv's dtype")
        self._call("hb_qk_norm_rope_kv_write", self._p(q_out), self._p(qkv), _code(qkv),
                   self._i32(positions, "positions"), self._p(table), rotary_dim,
                   table.shape[0] if table is not None else 0, self._p(q_weight), self._p(k_weight),
                   _code(q_weight) if q_weight is not None else 0, ctypes.c_float(eps), ctypes.c_float(offset),
                   self._p(kv), self._i32(write_index, "write_index"), kv.shape[0] if kv is not None else 0,
                   kv.shape[3] if kv is not None else 1, t, heads, kv_heads, head_dim)

    def qkv_rope(self, q_out, x, weight, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                 write_index, heads, kv_heads, head_dim) -> bool:
        """The product x · weightᵀ with qk_norm_rope_kv_write folded into its epilogue, for the few rows of a decode
        step (one kernel instead of two). False, with nothing done, where that kernel does not apply: more than
        SKINNY_ROWS rows, another dtype, a head size other than 32, 64 or 128, a partial rotation or none."""
        scaled, x = (x, x.y) if hasattr(x, "ss") else (None, x)      # rows that lack their norm's scale (parts.base.Scaled)
        t, k = x.shape
        wide = x.dtype == torch.bfloat16 and self._wide_takes(t, weight, scaled.ss.shape[1] if scaled else None)
        if not self.fused_qkv or x.dtype != torch.bfloat16 or (t > (self.MID_ROWS if self.mid else self.SKINNY_ROWS) and not wide) or k % 8 or table is None \
                or head_dim not in (32, 64, 128) or rotary_dim != head_dim or (q_weight is None) != (k_weight is None):
            return False
        self._check(q_out, x, weight, positions, table, q_weight, k_weight, kv, write_index)
        if weight.shape != ((heads + 2 * kv_heads) * head_dim, k) or weight.dtype != x.dtype \
                or q_out.shape != (t, heads, head_dim) or q_out.dtype != x.dtype:
            raise KernelError("qkv_rope: w must be [(heads + 2 kv_heads) head_dim, k] and q_out [tokens, heads, head_dim], bfloat16")
        if table.dtype != torch.float32 or table.shape[1] != head_dim:
            raise KernelError("qkv_rope: the rotation table must be float32 [positions, head_dim]")
        if kv is not None and (kv.dtype != x.dtype or kv.shape[1:3] != (2, kv_heads) or kv.shape[4] != head_dim):
            raise KernelError("qkv_rope: kv must be [pages, 2, kv_heads, page_size, head_dim], bfloat16")
        if q_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("qkv_rope: the two norm weights must have one dtype")
        if wide:
            self._call("hb_qkv_rope_skinny32", self._p(q_out), self._p(x), self._p(weight), t, k,
                       self._i32(positions, "positions"), self._p(table), table.shape[0], self._p(q_weight), self._p(k_weight),
                       int(q_weight is not None and q_weight.dtype == torch.float32), ctypes.c_float(eps),
                       ctypes.c_float(offset), self._p(kv), self._i32(write_index, "write_index"),
                       kv.shape[0] if kv is not None else 0, kv.shape[3] if kv is not None else 1, heads, kv_heads, head_dim,
                       self._p(scaled.ss) if scaled else None, scaled.ss.shape[0] if scaled else 0,
                       ctypes.c_float(scaled.eps if scaled else 0.0), scaled.dim if scaled else 0)
            return True
        if t > self.SKINNY_ROWS or self._mid_takes(t, weight, 2):
            self.mid_launches += 1
            self._call("hb_qkv_rope_mid", self._p(q_out), self._p(x), self._p(weight), t, k,
                       self._i32(positions, "positions"), self._p(table), table.shape[0], self._p(q_weight), self._p(k_weight),
                       int(q_weight is not None and q_weight.dtype == torch.float32), ctypes.c_float(eps),
                       ctypes.c_float(offset), self._p(kv), self._i32(write_index, "write_index"),
                       kv.shape[0] if kv is not None else 0, kv.shape[3] if kv is not None else 1, heads, kv_heads, head_dim,
                       self._p(scaled.ss) if scaled else None, scaled.ss.shape[0] if scaled else 0,
                       scaled.ss.shape[1] if scaled else 0, ctypes.c_float(scaled.eps if scaled else 0.0),
                       scaled.dim if scaled else 0, int(self.mid_split))
            return True
        if self._pending and scaled is not None and self._chains(t, k, x, weight):
            # the product that made these rows is still queued: this one joins it as a plain product, so that the
            # weights of both stream through one kernel, and the norm, rotation and cache write run behind it
            qkv = torch.empty((t, weight.shape[0]), dtype=torch.bfloat16, device=self.device)
            self._queue(w=weight, x=x, out=qkv, mode=0, n=weight.shape[0], scaled=scaled)
            self.qk_norm_rope_kv_write(q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                                       write_index, heads, kv_heads, head_dim)
            return True
        self._call("hb_qkv_rope_skinny_linked", self._p(q_out), self._p(x), self._p(weight), t, k,
                   self._i32(positions, "positions"), self._p(table), table.shape[0], self._p(q_weight), self._p(k_weight),
                   int(q_weight is not None and q_weight.dtype == torch.float32), ctypes.c_float(eps),
                   ctypes.c_float(offset), self._p(kv), self._i32(write_index, "write_index"),
                   kv.shape[0] if kv is not None else 0, kv.shape[3] if kv is not None else 1, heads, kv_heads, head_dim,
                   self._p(scaled.ss) if scaled else None, scaled.ss.shape[0] if scaled else 0,
                   ctypes.c_float(scaled.eps if scaled else 0.0), scaled.dim if scaled else 0)
        return True

    def paged_attention(self, out, q, kv, block_table, rows, scale, window) -> None:
        self._check(out, q, kv, block_table, rows.row_slot, rows.query_start, rows.kv_len)
        t, heads, head_dim = q.shape
        if out.shape != q.shape or kv.dtype != q.dtype or out.dtype != q.dtype or kv.shape[4] != head_dim:
            raise KernelError("paged_attention: out and q [tokens, heads, head_dim], kv [pages, 2, kv_heads, page_size, "
                              "head_dim], one dtype")
        fast = q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and self.attention_bf16 == "fast"
        if not fast:
            return self._attention_generic(out, q, kv, block_table, rows, scale, window)
        kv_heads = kv.shape[2]
        common = (self._i32(block_table, "block_table"), block_table.shape[1], self._i32(rows.row_slot, "row_slot"),
                  self._i32(rows.query_start, "query_start"), self._i32(rows.kv_len, "kv_len"))
        sizes = (heads, kv_heads, head_dim, kv.shape[0], kv.shape[3], ctypes.c_float(scale), int(window))
        if rows.n_decode:
            splits = self.decode_splits(rows.n_decode, heads, kv_heads, rows.max_kv)
            mode = self._decode_mode_of(rows)
            if splits > 1 and mode == "balanced" and rows.n_decode <= self.BALANCED_ROWS:
                pairs = rows.n_decode * kv_heads * (-(-(heads // kv_heads) // 16))
                slots = self.sms * (1 if head_dim > 128 else 3)       # CTAs of this kernel that one wave holds
                if 2 * pairs <= slots:                                # a whole number of CTAs per (row, kv head): rows of
                    slots = pairs * (slots // pairs)                  # equal length are then cut at their own ends only
                # (with more than half a wave of pairs that rounding would leave one CTA a pair and up to half of the
                # GPU idle: 29 rows of 8 kv heads, 83 µs against 50 µs with equal cuts)
                ctas = self.decode_ctas or max(1, min(slots, pairs * (-(-rows.max_kv // 64)) // 2))
                floats = (ctas + pairs) * min(16, heads // kv_heads) * (head_dim + 2)
                scratch = torch.empty(floats, dtype=torch.float32, device=self.device)
                self._call("hb_attention_decode_bf16_balanced", self._p(out), self._p(scratch), self._p(q), self._p(kv),
                           *common, rows.n_decode, *sizes, ctas)
            elif splits > 1 and (few := self.decode_cluster_splits(rows.n_decode, heads, kv_heads, head_dim,
                                                                   rows.max_kv, splits)):
                self._call("hb_attention_decode_bf16_cluster", self._p(out), self._p(q), self._p(kv), *common,
                           rows.n_decode, *sizes, few)
            else:
                floats = rows.n_decode * heads * splits * (head_dim + 2) if splits > 1 else 0
                scratch = torch.empty(floats, dtype=torch.float32, device=self.device) if floats else None
                self._call("hb_attention_decode_bf16", self._p(out), self._p(scratch), self._p(q), self._p(kv), *common,
                           rows.n_decode, *sizes, splits)
        if rows.n_rows > rows.n_decode:
            if self.prefill_attention == "tcgen05" and head_dim == 128 and kv.shape[3] % 64 == 0:
                tile_q, tiles = 256, self._query_tiles(rows, 256)
                if self.prefill_tile == 128 or (self.prefill_tile is None and 4 * heads * tiles < 3 * self.sms):              # tiles of 256 queries would leave SMs idle: one group of
                    tile_q, tiles = 128, self._query_tiles(rows, 128)   # 128 a CTA, twice the CTAs
                self._call("hb_attention_prefill_tcgen05", self._p(out), self._p(q), self._p(kv), *common,
                           rows.n_decode, rows.n_rows, tiles, t, *sizes, tile_q)
            else:
                self._call("hb_attention_prefill_bf16", self._p(out), self._p(q), self._p(kv), *common, rows.n_decode,
                           rows.n_rows, self._query_tiles(rows, 64), *sizes)

    KV_BUCKET_MIN = 512                       # the smallest number of keys a captured decode launch is planned for

    def attention_capture_plan(self, rows, max_model_len: int):
        """For a step that runs as a CUDA graph: what of the attention's launch plan a captured launch keeps, as a
        hashable key, pinned on `rows` so that every layer's launch is planned with it. The keys of a row are cut for
        a power-of-two bucket of the longest row (a graph of that bucket serves every batch whose longest row fits
        it; planning every graph for the longest request the engine takes would cut 2,000-token rows like 8,000-token
        ones), the one-token rows' keys are shared out in the mode their lengths call for, and rows of several tokens
        get the most query tiles any cut of their tokens into that many rows can have (tiles beyond a step's own exit
        at once)."""
        lens = rows.host_kv_len
        bucket = self.KV_BUCKET_MIN
        longest = int(lens.max()) if lens is not None and len(lens) else max_model_len
        while bucket < longest:
            bucket *= 2
        bucket = min(bucket, max(max_model_len, longest))
        mode = self.decode_mode(lens[:rows.n_decode] if lens is not None else None) if rows.n_decode else None
        rows.max_kv = bucket
        rows.plan["mode"] = mode
        portions, tokens = rows.n_rows - rows.n_decode, rows.n_tokens - rows.n_decode
        for size in (64, 128, 256):
            rows.plan[size] = tokens // size + portions
        return mode, bucket

    # Every layer of a step asks the same questions about the step's rows: the answers are kept on the rows.
    def _decode_mode_of(self, rows) -> str:
        plan = rows.plan
        if "mode" not in plan:
            lens = rows.host_kv_len[:rows.n_decode] if rows.host_kv_len is not None else None
            plan["mode"] = self.decode_mode(lens)
        return plan["mode"]

    @staticmethod
    def _query_tiles(rows, size: int) -> int:
        """Tiles of `size` queries over the rows that bring several tokens."""
        plan = rows.plan
        if size not in plan:
            qs = rows.host_query_start
            plan[size] = sum((int(qs[b + 1]) - int(qs[b]) + size - 1) // size for b in range(rows.n_decode, rows.n_rows))
        return plan[size]

    BALANCED_ROWS = 256                       # rows the balanced decode kernel takes (its prefix array)

    def decode_mode(self, kv_lens) -> str:
        """"balanced" or "splits" for decode rows that hold `kv_lens` tokens (host values; None: unknown). Equal cuts
        are a little faster while rows are alike (no walk crosses a row's end, one table read less before the first
        tile); one long row among short ones is where they lose: measured at 32 kv-head-8 rows, one of 8,192 tokens
        and 31 of 500, 36 µs against 56 µs."""
        if self.decode_attention != "auto":
            return self.decode_attention
        if kv_lens is None or len(kv_lens) < 2:
            return "splits"
        longest, total = int(max(kv_lens)), int(sum(int(v) for v in kv_lens))
        return "balanced" if longest >= 4096 and longest * len(kv_lens) >= 8 * total else "splits"

    def _split_cost(self, rows: int, heads: int, kv_heads: int, max_kv: int, splits: int) -> int:
        """Waves x (tiles a CTA walks + 1 for its start): what a launch of `splits` parts a row costs, in tile times."""
        ctas, tiles, slots = rows * kv_heads * (-(-(heads // kv_heads) // 16)), -(-max_kv // 64), 3 * self.sms
        return -(-ctas * splits // slots) * (-(-tiles // splits) + 1)

    def decode_splits(self, rows: int, heads: int, kv_heads: int, max_kv: int, most: int = 64) -> int:
        """Parts the keys of a decode row are cut into. Three CTAs fit an SM; a launch of `ctas * parts` CTAs runs in
        waves of 3 x SMs, each CTA walking its share of the longest row's 64-key tiles plus a fixed start-up of
        about one tile. The number of parts (1 to `most`) with the least waves x (tiles + 1) wins. It is a function of
        the batch's size and the longest length only, as the reference plans its splits
        (plugins/holon_plugins/kernels/triton_attn/plugin.py:40-96)."""
        key = (rows, heads, kv_heads, -(-max_kv // 64), most)
        if key not in self._splits:
            tiles = key[3]
            self._splits[key] = min(range(1, max(1, min(most, tiles)) + 1),
                                    key=lambda s: (self._split_cost(rows, heads, kv_heads, max_kv, s), s))
        return self._splits[key]

    MERGE_KERNEL_TILES = 6                    # what the second kernel and its scratch cost, in 64-key tile times

    def decode_cluster_splits(self, rows: int, heads: int, kv_heads: int, head_dim: int, max_kv: int, splits: int) -> int:
        """The number of splits (2 to 16) that merge inside the kernel as one thread-block cluster per (row, kv head),
        or 0 where `splits` parts and the merge kernel are the better plan. A cluster is taken only while all of them
        run at once (over several waves clusters leave holes: at 64 rows 16.6 ms a step against 15.4 ms with the merge
        kernel; the runtime says how many clusters of each size fit, and from 12 CTAs a cluster that is fewer than
        the CTA slots suggest); of those sizes the one whose CTAs walk the fewest tiles wins. Measured at 8,192 keys
        and 8 kv heads of 128, that cluster against the best number of splits with the merge kernel: 1 row 20.5 µs
        (16 CTAs) / 21.4, 3 rows 27.7 (15) / 29.7, 6 rows 38.9 (8) / 44.0, 8 rows 49.2 (6) / 56.2, 16 rows 87.0 (3) /
        93.2, 24 rows 122.9 (2) / 138.2; from 32 rows on no size fits one wave."""
        if not self.decode_cluster:
            return 0
        key = ("cluster", rows, heads, kv_heads, head_dim, -(-max_kv // 64), splits)
        if key not in self._splits:
            pairs, tiles = rows * kv_heads * (-(-(heads // kv_heads) // 16)), -(-max_kv // 64)
            fitting = [s for s in range(2, min(16, tiles) + 1) if pairs <= self._cluster_capacity(head_dim, s)]
            best = min(fitting, key=lambda s: (-(-tiles // s), s), default=0)
            merged = self._split_cost(rows, heads, kv_heads, max_kv, splits) + self.MERGE_KERNEL_TILES
            self._splits[key] = best if best and -(-tiles // best) + 1 <= merged else 0
        return self._splits[key]

    def _cluster_capacity(self, head_dim: int, splits: int) -> int:
        key = ("capacity", -(-head_dim // 64) if head_dim <= 128 else 3, splits)
        if key not in self._splits:
            fn = self.lib.hb_attention_decode_cluster_capacity
            fn.restype = ctypes.c_int
            self._splits[key] = int(fn(int(head_dim), int(splits)))
        return self._splits[key]

    def _attention_generic(self, out, q, kv, block_table, rows, scale, window) -> None:
        t, heads, head_dim = q.shape
        self._call("hb_attention_generic", self._p(out), self._p(q), self._p(kv), _code(q),
                   self._i32(block_table, "block_table"), block_table.shape[1], self._i32(rows.row_slot, "row_slot"),
                   self._i32(rows.query_start, "query_start"), self._i32(rows.kv_len, "kv_len"), rows.n_rows, t,
                   heads, kv.shape[2], head_dim, kv.shape[0], kv.shape[3], ctypes.c_float(scale), int(window))

    # ---- the residual sum and the next norm inside the product that ends a part (decode steps)
    def can_link(self, rows: int, hidden: int, norm) -> bool:
        """Whether a product of `rows` rows may add itself into the stream and leave `norm`'s rows unscaled for the
        next product: both run in the weight-streaming kernels, which take SKINNY_ROWS rows and, on clusters, MID_ROWS."""
        w = getattr(norm, "weight", None)
        most = self.MID_ROWS if self.mid else self.WIDE_ROWS if self.skinny32 else self.SKINNY_ROWS
        return self.fused_norm and 0 < rows <= most and hidden % 8 == 0 and w is not None \
            and w.tensor.dtype in (torch.bfloat16, torch.float32) and w.tensor.shape == (hidden,)

    def linear_link(self, h, x, weight, norm_weight, eps: float, offset: float):
        """h [m, n] (float32) += bfloat16(x · weightᵀ) and, returned as parts.base.Scaled, the new h times
        (norm_weight + offset) in bfloat16 with the partial sums of squares its RMSNorm still needs. None, with
        nothing done, where the kernel does not apply (another dtype, k no multiple of 8, more rows)."""
        from ..parts.base import Scaled
        m, k = x.shape
        n = weight.shape[0]
        wide = self._wide_takes(m, weight)
        if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or h.dtype != torch.float32 or k % 8 \
                or not (0 < m <= (self.MID_ROWS if self.mid else self.SKINNY_ROWS) or wide) or tuple(h.shape) != (m, n) \
                or weight.shape != (n, k):
            return None
        self._check(h, x, weight, norm_weight)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=self.device)
        if wide:
            ss = torch.empty((-(-n // 16), self.WIDE_ROWS), dtype=torch.float32, device=self.device)
            self._call("hb_gemm_bf16_skinny32", self._p(y), 0, self._p(x), self._p(weight), m, n, k, 3, 0, self._p(h),
                       self._p(norm_weight), int(norm_weight.dtype == torch.float32), ctypes.c_float(offset), self._p(ss),
                       None, 0, ctypes.c_float(0.0), 0)
            return Scaled(y, ss, float(eps), n)
        if m > self.SKINNY_ROWS:
            self.mid_launches += 1
            ss = torch.empty((-(-n // 256), self.MID_ROWS), dtype=torch.float32, device=self.device)
            self._call("hb_gemm_bf16_mid", self._p(y), 0, self._p(x), self._p(weight), m, n, k, 3, 0, self._p(h),
                       self._p(norm_weight), int(norm_weight.dtype == torch.float32), ctypes.c_float(offset), self._p(ss),
                       None, 0, 0, ctypes.c_float(0.0), 0, int(self.mid_split))
            return Scaled(y, ss, float(eps), n)
        parts = -(-n // 16)
        ss = torch.empty((parts, 16), dtype=torch.float32, device=self.device)
        if self._chains(m, k, x, weight, y) and norm_weight.dtype in (torch.bfloat16, torch.float32):
            self._queue(w=weight, x=x, out=y, mode=3, n=n, h=h, next_weight=norm_weight, next_offset=offset, ss_out=ss)
            return Scaled(y, ss, float(eps), n)
        self._call("hb_gemm_bf16_skinny_linked", self._p(y), 0, self._p(x), self._p(weight), m, n, k, 3, 0, self._p(h),
                   self._p(norm_weight), int(norm_weight.dtype == torch.float32), ctypes.c_float(offset), self._p(ss),
                   None, 0, ctypes.c_float(0.0), 0)
        return Scaled(y, ss, float(eps), n)

    def _scaled_product(self, out, x, weight, mode: int, inter: int) -> None:
        """A product whose x is parts.base.Scaled: the weight-streaming kernel applies the row scale to its sums."""
        y = x.y
        self._check(out, y, x.ss, weight)
        m, k = y.shape
        if m > self.MID_ROWS or k % 8 or y.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.shape[1] != k:
            raise KernelError("a product of unscaled rows takes up to MID_ROWS bfloat16 rows of a multiple of 8 columns")
        if self._wide_takes(m, weight, x.ss.shape[1]):
            return self._call("hb_gemm_bf16_skinny32", self._p(out), int(out.dtype == torch.float32), self._p(y),
                              self._p(weight), m, weight.shape[0], k, mode, inter, None, None, 0, ctypes.c_float(0.0), None,
                              self._p(x.ss), x.ss.shape[0], ctypes.c_float(x.eps), x.dim)
        if m > self.SKINNY_ROWS or self._mid_takes(m, weight, mode):
            self.mid_launches += 1
            return self._call("hb_gemm_bf16_mid", self._p(out), int(out.dtype == torch.float32), self._p(y), self._p(weight),
                              m, weight.shape[0], k, mode, inter, None, None, 0, ctypes.c_float(0.0), None, self._p(x.ss),
                              x.ss.shape[0], x.ss.shape[1], ctypes.c_float(x.eps), x.dim, int(self.mid_split))
        if self._chains(m, k, y, weight) and out.dtype in (torch.bfloat16, torch.float32) and (mode == 0 or out.dtype == torch.bfloat16):
            self._queue(w=weight, x=x, out=out, mode=mode, n=weight.shape[0], inter=inter, scaled=x)
            return
        self._call("hb_gemm_bf16_skinny_linked", self._p(out), int(out.dtype == torch.float32), self._p(y), self._p(weight),
                   m, weight.shape[0], k, mode, inter, None, None, 0, ctypes.c_float(0.0), None, self._p(x.ss),
                   x.ss.shape[0], ctypes.c_float(x.eps), x.dim)

    def linear(self, out, x, weight) -> None:
        if hasattr(x, "ss"):                             # rows that lack their norm's scale (parts.base.Scaled)
            if weight.shape[1] != x.shape[1] or out.shape != (x.shape[0], weight.shape[0]):
                raise KernelError(f"linear: x {tuple(x.shape)} · w {tuple(weight.shape)}ᵀ -> out {tuple(out.shape)} do not fit")
            return self._scaled_product(out, x, weight, 0, 0)
        self._check(out, x, weight)
        m, k = x.shape
        n = weight.shape[0]
        if weight.shape != (n, k) or out.shape != (m, n) or x.dtype != weight.dtype:
            raise KernelError(f"linear: x {tuple(x.shape)} · w {tuple(weight.shape)}ᵀ -> out {tuple(out.shape)} do not fit")
        if self._pending:
            if self._chains(m, k, x, weight) and out.data_ptr() % 16 == 0 and self._pending[0][2] == m:
                self._queue(w=weight, x=x, out=out, mode=0, n=n)   # (the last of a run of products: with them, then out)
                return self.flush()
            self.flush()
        if x.dtype == torch.float32:
            if out.dtype != torch.float32:
                raise KernelError("linear: a float32 product writes float32")
            self._call("hb_gemm_f32", self._p(out), self._p(x), self._p(weight), m, n, k)
        elif m <= self.SKINNY_ROWS and k % 8 == 0:       # decode steps: bound by reading the weight once
            self._call("hb_gemm_bf16_skinny", self._p(out), int(out.dtype == torch.float32), self._p(x),
                       self._p(weight), m, n, k, 0, 0)
        elif self.gemm == "tcgen05" and k % 8 == 0:      # the hand-written tensor-memory kernel in place of the library
            self.linear_tcgen05(out, x, weight)
        elif out.dtype == torch.float32:                 # the head: bfloat16 operands, 32-bit logits
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, weight.t(), out=out)

    SKINNY_ROWS = 16
    MID_ROWS = 64                             # rows the clustered tcgen05 products take (csrc/gemm_mid.cu)

    def linear_mid(self, out, x, weight, swiglu: bool = False, split: int = 0) -> None:
        """The product (or SwiGLU's silu(gate) · up) of up to MID_ROWS bfloat16 rows on csrc/gemm_mid.cu, whatever the
        table's own choice for these sizes would be (tests, microbench); `split`: the cluster size (0: chosen)."""
        self._check(out, x, weight)
        m, k = x.shape
        n = weight.shape[0]
        inter = n // 2 if swiglu else 0
        if weight.shape != (n, k) or out.shape != (m, inter if swiglu else n) or x.dtype != torch.bfloat16 \
                or weight.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("linear_mid: bfloat16 x [m, k] and w [n, k]; out [m, n] (or [m, n / 2]) bfloat16 or float32")
        self.mid_launches += 1
        self._call("hb_gemm_bf16_mid", self._p(out), int(out.dtype == torch.float32), self._p(x), self._p(weight), m, n, k,
                   int(swiglu), inter, None, None, 0, ctypes.c_float(0.0), None, None, 0, 0, ctypes.c_float(0.0), 0, int(split))

    def linear_tcgen05(self, out, x, weight, swiglu: bool = False, pair: bool | None = None) -> None:
        """The product (or, with `swiglu`, SwiGLU's silu(gate) · up) on the hand-written tcgen05 / TMA / TMEM kernels:
        `pair` picks the one that puts two CTAs on a 256 x 256 tile (default: self.gemm_pair)."""
        self._check(out, x, weight)
        m, k = x.shape
        n = weight.shape[0]
        inter = n // 2 if swiglu else 0
        if weight.shape != (n, k) or out.shape != (m, inter if swiglu else n) or x.dtype != torch.bfloat16 \
                or weight.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("linear_tcgen05: bfloat16 x [m, k] and w [n, k]; out [m, n] (or [m, n / 2]) bfloat16 or float32")
        name = "hb_gemm_bf16_tcgen05_pair" if (self.gemm_pair if pair is None else pair) else "hb_gemm_bf16_tcgen05"
        self._call(name, self._p(out), int(out.dtype == torch.float32), self._p(x), self._p(weight), m, n, k,
                   int(swiglu), inter)

    def status(self) -> int:
        """0, or the code of a bounded wait inside a kernel that gave up: (place << 28) | (block + 1). A read of host
        memory, no synchronisation: it tells of every kernel that has finished (wait for the step's event first)."""
        return int(self._status_word[0])

    def clear_status(self) -> None:
        self._status_word[0] = 0

    def status_selftest(self, polls: int = 1000) -> None:
        """Enqueues a wait of `polls` polls on a barrier nobody arrives at: it runs out and `status()` turns non-zero."""
        self._call("hb_status_selftest", int(polls))

    def tcgen05_status(self) -> int:
        """0, or which bounded wait inside a kernel (a tcgen05 product or attention, the chained products) gave up
        (synchronises the device; clears the kernels' words and the host's). After a wait of the chained products gave
        up their barrier and flags are put back to zero, so that the next launch starts clean."""
        out = 0
        for name in ("hb_gemm_tcgen05_status", "hb_gemm_tcgen05_pair_status", "hb_attention_tcgen05_status",
                     "hb_gemm_chain_status", "hb_gemm_tickets_status", "hb_gemm_mid_status"):
            status = ctypes.c_uint(0)
            if getattr(self.lib, name)(ctypes.byref(status)):
                raise KernelError(self.lib.hb_last_error().decode())
            out = out or status.value
        self.clear_status()
        if out:
            self._chain_sync.zero_()
            self._chain_flags.zero_()
            self._ticket_state.zero_()
        return out

    def swiglu_gate_up(self, out, x, weight) -> None:
        """out [tokens, inter] = silu(x · gateᵀ) · (x · upᵀ) with gate's rows first in `weight` [2 inter, k]: for a
        few tokens one kernel with the activation in its epilogue, else the product and the activation kernel."""
        if hasattr(x, "ss"):                             # rows that lack their norm's scale (parts.base.Scaled)
            if weight.shape != (2 * out.shape[1], x.shape[1]) or out.shape[0] != x.shape[0] or out.dtype != torch.bfloat16:
                raise KernelError("swiglu_gate_up: x [tokens, k], weight [2 inter, k], out [tokens, inter], one dtype")
            return self._scaled_product(out, x, weight, 1, out.shape[1])
        self._check(out, x, weight)
        m, k = x.shape
        inter = out.shape[1]
        if weight.shape != (2 * inter, k) or out.shape[0] != m or not (out.dtype == x.dtype == weight.dtype):
            raise KernelError("swiglu_gate_up: x [tokens, k], weight [2 inter, k], out [tokens, inter], one dtype")
        if x.dtype == torch.bfloat16 and k % 8 == 0 and self._wide_takes(m, weight):
            return self._call("hb_gemm_bf16_skinny32", self._p(out), 0, self._p(x), self._p(weight), m, 2 * inter, k, 1, inter,
                              None, None, 0, ctypes.c_float(0.0), None, None, 0, ctypes.c_float(0.0), 0)
        if x.dtype == torch.bfloat16 and k % 8 == 0 and self._mid_takes(m, weight, 1):
            return self.linear_mid(out, x, weight, swiglu=True, split=self.mid_split)
        if x.dtype == torch.bfloat16 and m <= self.SKINNY_ROWS and k % 8 == 0:
            self._call("hb_gemm_bf16_skinny", self._p(out), 0, self._p(x), self._p(weight), m, 2 * inter, k, 1, inter)
            return
        if x.dtype == torch.bfloat16 and k % 8 == 0 and self.gemm != "cublas":
            # Measured at 24576 x 4096 against the library's product plus the activation kernel: by CTA pairs 66 us
            # against 74 at 256 rows, 280 against 317 at 2,048, 555 against 627 at 4,096, but 1,226 against 1,202 at
            # 8,192; one CTA a tile 59 against 66 at 128 rows; below about 100 rows the library wins (64 against 70).
            if self.gemm == "tcgen05" or 192 < m <= 6144:
                self.linear_tcgen05(out, x, weight, swiglu=True)
                return
            if 96 < m <= 192:
                self.linear_tcgen05(out, x, weight, swiglu=True, pair=False)
                return
        gate_up = torch.empty(m, 2 * inter, dtype=x.dtype, device=self.device)
        self.linear(gate_up, x, weight)
        self.silu_mul(out, gate_up)

    def feed_tokens(self, token_ids, last_tokens, rows, from_last) -> None:
        """token_ids[first token of row r] = last_tokens[slot of row r] for the rows whose `from_last` is set."""
        self._check(token_ids, last_tokens, rows.row_slot, rows.query_start, from_last)
        self._call("hb_feed_tokens", self._i32(token_ids, "token_ids"), self._i32(last_tokens, "last_tokens"),
                   self._i32(rows.row_slot, "row_slot"), self._i32(rows.query_start, "query_start"),
                   self._i32(from_last, "from_last"), rows.n_rows)

    def scatter_rows(self, table, slots, rows) -> None:
        """table[slots[i], :] = rows[i, :]: block-table rows that changed on the host, packed in the step's upload."""
        self._check(table, slots, rows)
        n, width = slots.shape[0], table.shape[1]
        if rows.shape[0] != n * width:
            raise KernelError(f"scatter_rows: {n} rows of {width} need {n * width} values, not {rows.shape[0]}")
        self._call("hb_scatter_rows", self._i32(table, "table"), self._i32(slots, "slots"), self._i32(rows, "rows"),
                   n, width, table.shape[0])

    def store_tokens(self, last_tokens, slots, tokens, n) -> None:
        """last_tokens[slots[i]] = tokens[i] for i < n."""
        self._check(last_tokens, slots, tokens)
        self._call("hb_store_tokens", self._i32(last_tokens, "last_tokens"), self._i32(slots, "slots"),
                   self._i32(tokens, "tokens"), int(n))

    def logprobs(self, chosen, top_ids, top, logits, tokens) -> None:
        """chosen [rows] float32: log softmax(logits)[tokens]; top_ids int32 / top float32 [rows, k]: the k most likely."""
        self._check(chosen, top_ids, top, logits, tokens)
        r, v = logits.shape
        k = top.shape[1]
        if logits.dtype != torch.float32 or chosen.dtype != torch.float32 or top.dtype != torch.float32 \
                or top_ids.dtype != torch.int32 or tokens.dtype != torch.int32:
            raise KernelError("logprobs: logits, chosen, top float32; top_ids, tokens int32")
        if chosen.shape[0] < r or tokens.shape[0] < r or top.shape != (r, k) or top_ids.shape != (r, k):
            raise KernelError("logprobs: chosen and tokens [rows], top_ids and top [rows, k]")
        self._call("hb_logprobs", self._p(chosen), self._p(top_ids), self._p(top), self._p(logits), self._p(tokens), r, v, k)

    def sample(self, tokens, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, position, filtered) -> None:
        self._check(tokens, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, position)
        r, v = logits.shape
        if logits.dtype != torch.float32 or tokens.dtype != torch.int32 or tokens.shape[0] < r:
            raise KernelError("sample: logits float32 [rows, vocab], tokens int32 [rows]")
        for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                            ("min_p", min_p, torch.float32), ("top_k", top_k, torch.int32),
                            ("seed_lo", seed_lo, torch.int32), ("seed_hi", seed_hi, torch.int32),
                            ("position", position, torch.int32)):
            if t.dtype != dt or t.shape[0] < r:
                raise KernelError(f"sample: {name} must be {dt} [rows]")
        self._call("hb_sample", self._p(tokens), self._p(logits), self._p(temperature), self._p(top_k),
                   self._p(top_p), self._p(min_p), self._p(seed_lo), self._p(seed_hi), self._p(position),
                   int(bool(filtered)), r, v)

"""Python face of the CUDA kernels: one function per kernel, taking torch CUDA tensors.

Every function checks dtypes, contiguity and sizes, then launches on the current
CUDA stream through the C ABI of the compiled library.  Nothing here computes on
the CPU or falls back to a library: a tensor that is not on a CUDA device, or a
library that cannot be built or loaded, raises ``KernelError``.

The library keeps small tables (tensor maps it has made, shared-memory allowances, the text of the
last error) without locks: one thread at a time may call into it, which is how the engine drives it.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..errors import KernelError
from . import build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_void_p = ctypes.c_void_p


_VP, _I, _F, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
# Argument types of the launchers on the model's path: with these declared, plain Python ints and floats go straight
# to C (a pointer would otherwise be cut to 32 bits, and wrapping every argument in a ctypes object costs microseconds).
_SIGNATURES = {
    "ferris_gemm_tcgen05": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _I, _VP, _VP, _VP],
    "ferris_norm_gemm_tcgen05": [_VP, _VP, _F, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_merge_gemm_tcgen05": [_VP, _I, _I, _I, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_qkv_rope_gemm_tcgen05": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _VP],
    "ferris_rotary_angles": [_VP, _VP, _VP, _I, _I, _VP],
    "ferris_rmsnorm": [_VP, _VP, _VP, _VP, _I, _I, _I, _F, _VP],
    "ferris_rope_cache_write": [_VP, _I, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_prefill_attention": [_VP, _I, _VP, _I, _VP, _VP, _LL, _VP, _I, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _F, _I, _VP],
    "ferris_decode_attention_rope": [_VP, _I, _VP, _I, _VP, _VP, _LL, _VP, _I, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I,
                                     _F, _I, _VP, _I, _VP],
    "ferris_gemm_argmax_tcgen05": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP, _VP],
    "ferris_gemm_skinny": [_VP, _I, _VP, _VP, _F, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ferris_gemm_skinny_takes": [_I, _I, _I, _I, _I],
    "ferris_embed_gather": [_VP, _I, _VP, _VP, _I, _I, _I, _VP, _VP],
}
_declared = False


def _lib():
    global _declared
    lib = build.load_library()
    if not _declared:
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int
        _declared = True
    return lib


def _dt(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def _stream() -> _c_void_p:
    """The raw handle of torch's current stream on the current device."""
    return _c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need(t: torch.Tensor, what: str, dtype=None, contiguous: bool = True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, found {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def _rows(t: torch.Tensor, what: str) -> tuple[int, int, int]:
    """(rows, cols, row stride) of a 2-D tensor whose rows are contiguous."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor (there is no CPU path)")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what} must be 2-D with contiguous rows, found shape {tuple(t.shape)} strides {t.stride()}")
    return t.shape[0], t.shape[1], t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


_launches = 0


def launch_count() -> int:
    """How many kernels this process has launched through this module."""
    return _launches


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    _launches += kernels
    if code != 0:
        msg = _lib().ferris_last_error().decode("utf-8", "replace")
        kind = "refused its arguments" if code < 0 else f"failed (CUDA error {code})"
        raise KernelError(f"{what} {kind}: {msg}")


def require_device() -> None:
    """Raise unless a CUDA device of compute capability 10.x is current and the library loads."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; this engine has no CPU path")
    arch = _lib().ferris_device_arch()
    if arch < 0:
        raise KernelError("cannot query the CUDA device: " + _lib().ferris_last_error().decode())
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a; the current device is sm_{arch}")


# ------------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out[t, :] = table[ids[t], :] as fp32.  ids int32 [T]; out fp32 [T, H]."""
    _need(table, "embedding table")
    _need(ids, "token ids", torch.int32)
    _need(out, "embedding output", torch.float32)
    T, H = out.shape
    if table.dim() != 2 or table.shape[1] != H or ids.numel() != T:
        raise KernelError(f"embed_gather: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    _check(
        _lib().ferris_embed_gather(_ptr(table), _dt(table, "embedding table"), _ptr(ids), _ptr(out), _c_int(T),
                                   _c_int(H), _c_int(table.shape[0]), _ptr(status), _stream()),
        "embed_gather",
    )


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            row_index: Optional[torch.Tensor] = None):
    """out[i] = rmsnorm(x[row_index[i]] or x[i]) * weight.  x fp32 [T, H]; weight fp32 [H]."""
    _need(x, "rmsnorm input", torch.float32)
    _need(weight, "rmsnorm weight", torch.float32)
    _need(out, "rmsnorm output")
    rows, H = out.shape
    if x.shape[1] != H or weight.numel() != H:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if row_index is not None:
        _need(row_index, "rmsnorm row index", torch.int32)
        if row_index.numel() != rows:
            raise KernelError("rmsnorm: one row index per output row is needed")
    elif x.shape[0] != rows:
        raise KernelError("rmsnorm: input and output row counts differ")
    _check(
        _lib().ferris_rmsnorm(x.data_ptr(), weight.data_ptr(), None if row_index is None else row_index.data_ptr(),
                              out.data_ptr(), _dt(out, "rmsnorm output"), rows, H, eps, _stream()),
        "rmsnorm",
    )


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              accumulate: bool = False):
    """out[t, n] (+)= sum_k x[t, k] w[n, k] + bias[n] with fp32 FMAs on the CUDA cores."""
    M, K, ldx = _rows(x, "gemm input")
    N, K2, ldw = _rows(w, "gemm weight")
    M2, N2, ldo = _rows(out, "gemm output")
    if K != K2 or M != M2 or N != N2 or x.dtype != w.dtype:
        raise KernelError(f"gemm: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm: bias length differs from the output width")
    _check(
        _lib().ferris_gemm_simt(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _dt(x, "gemm input"), _dt(out, "gemm output"),
                                _c_int(M), _c_int(N), _c_int(K), _c_int(ldx), _c_int(ldw), _c_int(ldo),
                                _c_int(1 if accumulate else 0), _stream()),
        "gemm",
    )


# Scratch of the tensor-core GEMM's K split: fp32 partials and per-tile counters.  Buffers only ever grow, and
# outgrown ones are kept alive, because a captured CUDA graph may still point at them.
_gemm_buffers: dict = {}
_gemm_retired: list = []
_GEMM_COUNTERS = 8192


def _gemm_scratch(device, floats: int, counters: int):
    key = str(device)
    entry = _gemm_buffers.get(key)
    if entry is None or entry[0].numel() < floats or entry[1].numel() < counters:
        if entry is not None:
            _gemm_retired.append(entry)
        size = max(floats, 1 << 20, 0 if entry is None else entry[0].numel())
        entry = (torch.empty(size, dtype=torch.float32, device=device),
                 torch.zeros(max(counters, _GEMM_COUNTERS), dtype=torch.int32, device=device))
        _gemm_buffers[key] = entry
    return entry


def tensor_core_gemm_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """bf16 operands with contiguous rows, K and the row strides multiples of 8, 16-byte aligned bases."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        return False
    K = x.shape[1]
    ldx = x.stride(0) if x.shape[0] > 1 else max(x.stride(0), K)
    ldw = w.stride(0) if w.shape[0] > 1 else max(w.stride(0), K)
    return (K % 8 == 0 and ldx % 8 == 0 and ldw % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (K <= 1 or (x.stride(1) == 1 and w.stride(1) == 1)))


_uses_clusters = None


def gemm_tcgen05(x, w, bias, out, mode: int, n_out: Optional[int] = None, up_row_offset: int = 0):
    """out = x w^T on the tcgen05 tensor cores.  mode 0: bf16 store (+bias); 1: fp32 store (+bias);
    2: fp32 out += ; 3: bf16 silu(x w[:N]^T) * (x w[up_row_offset:up_row_offset+N]^T)."""
    global _uses_clusters
    T, K, ldx = _rows(x, "gemm input")
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    if n_out is not None and n_out != N:
        raise KernelError("gemm: output width differs from what was asked")
    want_dtype = torch.bfloat16 if mode in (0, 3) else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype:
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}, mode {mode}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm: bias length differs from the output width")
    lib = _lib()
    if _uses_clusters is None:
        _uses_clusters = bool(lib.ferris_gemm_uses_clusters())
    scratch = cnt = None
    if not _uses_clusters:
        # K splits that add up through global memory need scratch and counters
        bt, splits, floats, counters = _c_int(), _c_int(), ctypes.c_longlong(), _c_int()
        lib.ferris_gemm_tcgen05_plan(_c_int(T), _c_int(N), _c_int(K), _c_int(2 if mode == 3 else 1), ctypes.byref(bt),
                                     ctypes.byref(splits), ctypes.byref(floats), ctypes.byref(counters))
        if splits.value > 1:
            scratch, cnt = _gemm_scratch(x.device, floats.value, counters.value)
    _check(
        lib.ferris_gemm_tcgen05(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(),
                                mode, T, N, K, ldx, ldw, ldo, rows_w, up_row_offset,
                                None if scratch is None else scratch.data_ptr(), None if cnt is None else cnt.data_ptr(),
                                _stream()),
        "tensor-core gemm",
    )


def gemm_plan(tokens: int, outputs: int, k: int, accumulators: int = 1) -> tuple[int, int]:
    """How the short-step tcgen05 kernel would cut a product: (token tile, K splits)."""
    bt, splits, floats, counters = _c_int(), _c_int(), ctypes.c_longlong(), _c_int()
    _lib().ferris_gemm_tcgen05_plan(_c_int(tokens), _c_int(outputs), _c_int(k), _c_int(accumulators), ctypes.byref(bt),
                                    ctypes.byref(splits), ctypes.byref(floats), ctypes.byref(counters))
    return bt.value, splits.value


def gemm_argmax(x, w, out_token, out_prob, scratch):
    """out_token[t] = the lowest index among the greatest of (x w^T)[t, :], out_prob[t] = its softmax probability
    (may be None): the output head of rows that all take their greatest logit, on the tcgen05 tensor cores, without
    storing the logits.  At most 128 rows; ``scratch``: fp32, ``gemm_argmax_scratch_floats`` long."""
    T, K, ldx = _rows(x, "gemm input")
    N, K2, ldw = _rows(w, "gemm weight")
    if K != K2 or T > 128 or not tensor_core_gemm_takes(x, w):
        raise KernelError(f"product + argmax: x {tuple(x.shape)}, w {tuple(w.shape)} are not taken")
    _need(out_token, "tokens", torch.int32)
    if out_prob is not None:
        _need(out_prob, "probabilities", torch.float32)
    _need(scratch, "scratch", torch.float32)
    if out_token.numel() != T or (out_prob is not None and out_prob.numel() != T) \
            or scratch.numel() < gemm_argmax_scratch_floats(T, N):
        raise KernelError("product + argmax: one token (and probability) per row and enough scratch are needed")
    _check(
        _lib().ferris_gemm_argmax_tcgen05(x.data_ptr(), w.data_ptr(), out_token.data_ptr(),
                                          None if out_prob is None else out_prob.data_ptr(), T, N, K, ldx, ldw, N,
                                          scratch.data_ptr(), _stream()),
        "product + argmax",
    )


def gemm_argmax_scratch_floats(rows: int, outputs: int) -> int:
    return 4 * rows * ((outputs + 127) // 128)


GREEDY_HEAD_MAX_ROWS = 96


def greedy_head(y, w, out_token, out_prob, workspace):
    """The output head and greedy sampling of the rows ``y`` [n, H] in one: out_token int32 [n], out_prob fp32 [n].
    bf16 rows, at most 96: the product that stores no logits; anything else: logits into the workspace, then the
    sampling kernel's greedy rows.  The same tokens and probabilities either way (up to the rounding of the sums).
    (The product's epilogue reduces over the 128 outputs of a tile, which lie across the lanes of its warps, with
    three warp reductions a token.  With three of its CTAs to an SM that hides behind the weights' way in: measured
    inside the decode step of the 0.5B sizes against stored logits and the sampling kernel, ms a step at 17 / 24 / 48 /
    64 / 96 / 128 rows: 1.212 / 1.260 / 1.633 / 1.733 / 2.382 / 2.492 against 1.227 / 1.276 / 1.638 / 1.743 / 2.420 /
    2.487.)"""
    n, V = y.shape[0], w.shape[0]
    if n <= GREEDY_HEAD_MAX_ROWS and tensor_core_gemm_takes(y, w):
        scratch = workspace.get("argmax_tiles", (gemm_argmax_scratch_floats(n, V),), torch.float32)
        gemm_argmax(y, w, out_token, out_prob, scratch)
        return
    logits = workspace.get("logits", (n, V), torch.float32)
    gemm(y, w, None, logits)
    sample(logits, out_token, out_prob)


GEMM_PAIRS_NONE, GEMM_PAIRS_ALL, GEMM_PAIRS_SWIGLU = 0, 1, 2


def set_gemm_pairs(which=GEMM_PAIRS_SWIGLU) -> None:
    """Which products of long steps (more than 128 tokens) run on pairs of CTAs that share one 256-row MMA
    (cta_group::2): none, all, or the gate / up product only (the default, also of the library: see the
    measurements beside ferris_gemm_pair_enabled in csrc/gemm_tcgen05.cu).  True / False mean all / none."""
    _lib().ferris_set_gemm_pair(_c_int(int(which)))


def set_gemm_long_min(tokens: int = 0) -> None:
    """From how many tokens on a product runs the token-major kernel (never below 128); 0: the library's default."""
    _lib().ferris_set_gemm_long_min(_c_int(int(tokens)))


class LazyRMSNorm:
    """The RMSNorm of the residual rows ``h`` that has not been computed yet.  A matrix product that can form
    it on its way (``gemm`` / ``gemm_swiglu`` for short bf16 steps) takes it as its input and no norm kernel
    runs; everyone else calls ``materialize()`` and gets the normed rows, computed once."""

    def __init__(self, h: torch.Tensor, weight: torch.Tensor, eps: float, out_buffer: torch.Tensor):
        self.h, self.weight, self.eps, self._out, self._done = h, weight, float(eps), out_buffer, False

    @property
    def shape(self):
        return self._out.shape

    @property
    def dtype(self):
        return self._out.dtype

    def materialize(self) -> torch.Tensor:
        if not self._done:
            rmsnorm(self.h, self.weight, self.eps, self._out)
            self._done = True
        return self._out


def _norm_gemm_takes(x: "LazyRMSNorm", w: torch.Tensor, accs: int) -> bool:
    """Whether the short-step kernel can form the norm itself: bf16, at most 16 tokens, and a K split that
    leaves all of a CTA's slices resident at once."""
    T, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or T > 16 or K % 8 or x._done:
        return False
    if not (x.h.is_cuda and x.h.dtype == torch.float32 and x.h.is_contiguous() and x.h.data_ptr() % 16 == 0
            and x.weight.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0):
        return False
    return bool(_lib().ferris_gemm_tcgen05_builds_tokens(_c_int(T), _c_int(w.shape[0] // accs), _c_int(K), _c_int(accs)))


def norm_gemm_tcgen05(x: "LazyRMSNorm", w, bias, out, mode: int, up_row_offset: int = 0):
    """out = rmsnorm(h) w^T in one kernel (modes as gemm_tcgen05)."""
    T, K = x.shape
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    want_dtype = torch.bfloat16 if mode in (0, 3) else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype:
        raise KernelError(f"norm + gemm: h {tuple(x.h.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
    _check(
        _lib().ferris_norm_gemm_tcgen05(x.h.data_ptr(), x.weight.data_ptr(), x.eps, w.data_ptr(),
                                        None if bias is None else bias.data_ptr(), out.data_ptr(), mode, T, N, K, ldw,
                                        ldo, rows_w, up_row_offset, _stream()),
        "norm + gemm",
    )


class LazySplitMerge:
    """The attention rows of a single-token step whose key ranges (splits) have not been merged yet: the
    partial results lie in ``scratch``.  A matrix product that can merge them on its way (``gemm`` for short
    bf16 steps) takes this as its input and no merge kernel runs; everyone else calls ``materialize()``."""

    def __init__(self, scratch: torch.Tensor, out_buffer: torch.Tensor, num_heads: int, head_dim: int, splits: int):
        self.scratch, self._out, self._done = scratch, out_buffer, False
        self.num_heads, self.head_dim, self.splits = int(num_heads), int(head_dim), int(splits)

    @property
    def shape(self):
        return self._out.shape

    @property
    def dtype(self):
        return self._out.dtype

    def materialize(self) -> torch.Tensor:
        if not self._done:
            T, _, ldo = _rows(self._out, "attention output")
            _check(_lib().ferris_decode_merge(_ptr(self.scratch), _ptr(self._out), _c_int(ldo), _c_int(T),
                                              _c_int(self.num_heads), _c_int(self.head_dim), _c_int(self.splits), _stream()),
                   "decode merge")
            self._done = True
        return self._out


def _merge_gemm_takes(x: "LazySplitMerge", w: torch.Tensor) -> bool:
    """Whether the short-step kernel can merge the key ranges itself (the limits of the fused norm)."""
    T, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or T > 16 or x._done or w.shape[1] != K:
        return False
    if not (w.data_ptr() % 16 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and x.scratch.data_ptr() % 16 == 0):
        return False
    return bool(_lib().ferris_gemm_tcgen05_builds_tokens(_c_int(T), _c_int(w.shape[0]), _c_int(K), _c_int(1)))


def merge_gemm_tcgen05(x: "LazySplitMerge", w, bias, out, mode: int):
    """out (+)= merge(partial attention results) w^T in one kernel (modes 0-2 as gemm_tcgen05)."""
    T, K = x.shape
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    want_dtype = torch.bfloat16 if mode == 0 else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype or mode not in (0, 1, 2):
        raise KernelError(f"merge + gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
    _check(
        _lib().ferris_merge_gemm_tcgen05(_ptr(x.scratch), _c_int(x.num_heads), _c_int(x.head_dim), _c_int(x.splits),
                                         _ptr(w), _ptr(bias), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(ldw),
                                         _c_int(ldo), _c_int(rows_w), _stream()),
        "merge + gemm",
    )


def set_gemm_skinny(on: bool = True) -> None:
    """Steps of at most 16 tokens on the weight-stationary kernel of csrc/gemm_skinny.cu (True, the default, also
    of the library unless FERRIS_GEMM_SKINNY=0), or on the tcgen05 kernel with its K split over a cluster (False)."""
    _lib().ferris_set_gemm_skinny(_c_int(1 if on else 0))
    _skinny_shapes.clear()


_skinny_shapes: dict = {}


def gemm_skinny_enabled() -> bool:
    return bool(_lib().ferris_gemm_skinny_enabled())


def _skinny_takes(x, w, out, accs: int) -> bool:
    """Whether the skinny kernel takes this product: bf16, at most 16 tokens, K a multiple of 8, aligned rows, and a
    number of outputs that its plan covers (``x``: a tensor or a LazyRMSNorm that has not been computed)."""
    T, K = x.shape
    if T > 16 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 2 or w.shape[1] != K or K % 8:
        return False
    if w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16:
        return False
    if isinstance(x, LazyRMSNorm):
        if x._done or not (x.h.is_cuda and x.h.dtype == torch.float32 and x.h.is_contiguous() and x.h.data_ptr() % 16 == 0
                           and x.weight.data_ptr() % 16 == 0):
            return False
    elif not (x.dim() == 2 and x.is_cuda and x.stride(1) == 1 and (x.stride(0) % 8 == 0 or T == 1) and x.data_ptr() % 16 == 0):
        return False
    N = out.shape[1]
    formed = isinstance(x, LazyRMSNorm)  # rows that the kernel forms stand whole in shared memory; others may stream
    key = (T > 8, N, K, accs, formed)
    takes = _skinny_shapes.get(key)
    if takes is None:
        takes = bool(_lib().ferris_gemm_skinny_takes(T, N, K, accs, 0 if formed else 1))
        _skinny_shapes[key] = takes
    return takes


def gemm_skinny(x, w, bias, out, mode: int, up_row_offset: int = 0):
    """out (+)= x w^T (+ bias) for at most 16 tokens; ``x`` a bf16 tensor or a LazyRMSNorm (formed in the kernel).
    Modes as gemm_tcgen05."""
    T, K = x.shape
    rows_w, K2, ldw = _rows(w, "gemm weight")
    T2, N, ldo = _rows(out, "gemm output")
    want_dtype = torch.bfloat16 if mode in (0, 3) else torch.float32
    if K != K2 or T != T2 or out.dtype != want_dtype:
        raise KernelError(f"skinny gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}, mode {mode}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("gemm: bias length differs from the output width")
    lazy = isinstance(x, LazyRMSNorm)
    ldx = K if lazy else (x.stride(0) if T > 1 else max(x.stride(0), K))
    _check(
        _lib().ferris_gemm_skinny(None if lazy else x.data_ptr(), ldx, x.h.data_ptr() if lazy else None,
                                  x.weight.data_ptr() if lazy else None, x.eps if lazy else 0.0, w.data_ptr(),
                                  None if bias is None else bias.data_ptr(), out.data_ptr(), mode, T, N, K, ldw, ldo,
                                  rows_w, up_row_offset, _stream()),
        "skinny gemm",
    )


def _mode_of(out, accumulate: bool) -> int:
    return 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1)


def gemm(x, w, bias, out, accumulate: bool = False):
    """The matrix product of the model, out (+)= x w^T + bias: for bf16 operands the skinny kernel (at most 16
    tokens) or the tcgen05 kernels, the CUDA-core kernel for everything else (all of the 32-bit path).  ``x`` may
    be a LazyRMSNorm or a LazySplitMerge."""
    if isinstance(x, LazySplitMerge):
        if w.shape[0] == out.shape[1] and _merge_gemm_takes(x, w):
            merge_gemm_tcgen05(x, w, bias, out, 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1))
            return
        x = x.materialize()
    if w.shape[0] == out.shape[1] and x.shape[0] <= 16 and gemm_skinny_enabled() and _skinny_takes(x, w, out, 1):
        gemm_skinny(x, w, bias, out, _mode_of(out, accumulate))
        return
    if isinstance(x, LazyRMSNorm):
        if w.shape[0] == out.shape[1] and _norm_gemm_takes(x, w, 1):
            norm_gemm_tcgen05(x, w, bias, out, 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1))
            return
        x = x.materialize()
    if tensor_core_gemm_takes(x, w) and w.shape[0] == out.shape[1]:
        if accumulate:
            gemm_tcgen05(x, w, bias, out, 2)
        else:
            gemm_tcgen05(x, w, bias, out, 0 if out.dtype == torch.bfloat16 else 1)
        return
    gemm_simt(x, w, bias, out, accumulate)


_EPILOGUE_ACTIVATIONS = {"xielu": 1, "silu": 2, "relu2": 3}
_set_activation = None


def gemm_activation(x, w, out, kind: str, coefficients=(0.0, 0.0), params: Optional[torch.Tensor] = None):
    """out = a(x w^T): the plain feed-forward's up product with its activation.  bf16 on the weight-stationary kernel
    (at most 16 tokens) or the tcgen05 kernels of long steps: the activation is applied to the fp32 accumulator in
    the product's epilogue, before the one rounding to bf16
    (``coefficients``: for xIELU, (softplus(p), 1/2 + softplus(q)) as Python floats).  Anything else: the product,
    then the activation kernel with ``params`` (the two raw numbers on the device)."""
    global _set_activation
    if kind not in _EPILOGUE_ACTIVATIONS:
        raise KernelError(f"activation '{kind}' is not known")
    if out.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[0] == out.shape[1]:
        if _set_activation is None:
            _set_activation = _lib().ferris_gemm_set_activation
            _set_activation.argtypes = [_I, _F, _F]
            _set_activation.restype = None
        a, b = float(coefficients[0]), float(coefficients[1])
        code = _EPILOGUE_ACTIVATIONS[kind]
        try:  # the product that is launched next takes the activation; whatever happens, none is left behind
            if x.shape[0] <= 16 and gemm_skinny_enabled() and _skinny_takes(x, w, out, 1):
                _set_activation(code, a, b)
                gemm_skinny(x, w, None, out, 0)
                return
            if isinstance(x, LazyRMSNorm):
                x = x.materialize()
            # of the tcgen05 kernels only those of long steps apply an activation
            if tensor_core_gemm_takes(x, w) and _lib().ferris_gemm_tcgen05_fuses_activation(
                    _c_int(x.shape[0]), _c_int(out.shape[1]), _c_int(x.shape[1]), _c_int(out.stride(0)), _ptr(out)):
                _set_activation(code, a, b)
                gemm_tcgen05(x, w, None, out, 0)
                return
        finally:
            _set_activation(0, 0.0, 0.0)
    gemm(x, w, None, out)
    activation(out, out, kind, params)


def gemm_swiglu(x, gate_up_weight, out, workspace=None):
    """out [T, I] = silu(x Wg^T) * (x Wu^T) with gate_up_weight = [Wg; Wu] ([2I, K]).  bf16: one tensor-core
    kernel with two accumulators (the [T, 2I] intermediate never exists); otherwise a product and the SwiGLU kernel."""
    T, I = out.shape
    if gate_up_weight.shape[0] != 2 * I:
        raise KernelError(f"gemm_swiglu: weight {tuple(gate_up_weight.shape)} for {I} outputs")
    if T <= 16 and out.dtype == torch.bfloat16 and gemm_skinny_enabled() and _skinny_takes(x, gate_up_weight, out, 2):
        gemm_skinny(x, gate_up_weight, None, out, 3, up_row_offset=I)
        return
    if isinstance(x, LazyRMSNorm):
        if out.dtype == torch.bfloat16 and _norm_gemm_takes(x, gate_up_weight, 2):
            norm_gemm_tcgen05(x, gate_up_weight, None, out, 3, up_row_offset=I)
            return
        x = x.materialize()
    if tensor_core_gemm_takes(x, gate_up_weight) and out.dtype == torch.bfloat16:
        gemm_tcgen05(x, gate_up_weight, None, out, 3, up_row_offset=I)
        return
    if workspace is not None:
        gate_up = workspace.get("ffn_gate_up", (T, 2 * I), x.dtype)
    else:
        gate_up = torch.empty(T, 2 * I, dtype=x.dtype, device=x.device)
    gemm_simt(x, gate_up_weight, None, gate_up)
    swiglu(gate_up, out)


GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}
_set_gated = None


def gated_activation(gate_up: torch.Tensor, out: torch.Tensor, kind: str = "silu", limit: float = 0.0):
    """out[t, j] = f(gate_up[t, j], gate_up[t, I + j]): f = silu(g) u, gelu_tanh(g) u, or ("clamped_swish", with
    ``limit`` L) min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1); fp32 arithmetic."""
    T, I = out.shape
    T2, W2, ld = _rows(gate_up, "gated activation input")
    _need(out, "gated activation output", gate_up.dtype)
    if kind not in GATED_ACTIVATIONS or T2 != T or W2 != 2 * I:
        raise KernelError(f"gated activation '{kind}': input {tuple(gate_up.shape)}, output {tuple(out.shape)}")
    _check(_lib().ferris_gated_activation(_ptr(gate_up), _c_int(ld), _ptr(out), _c_int(_dt(out, "gated activation")), _c_int(T),
                                          _c_int(I), _c_int(GATED_ACTIVATIONS[kind]), _c_float(limit), _stream()),
           "gated activation")


def gemm_gated(x, gate_up_weight, out, kind: str = "silu", limit: float = 0.0, workspace=None):
    """out [T, I] = f(x Wg^T, x Wu^T) with gate_up_weight = [Wg; Wu] ([2I, K]) and f a gated activation (see
    ``gated_activation``).  "silu" is ``gemm_swiglu``.  The others in bf16: the weight-stationary kernel (at most 16
    tokens) and the tcgen05 kernels of long steps apply f to the two fp32 accumulators in their epilogue; anything else
    is the product followed by the activation kernel."""
    global _set_gated
    if kind == "silu":
        return gemm_swiglu(x, gate_up_weight, out, workspace)
    if kind not in GATED_ACTIVATIONS:
        raise KernelError(f"gated activation '{kind}' is not known ({', '.join(GATED_ACTIVATIONS)})")
    T, I = out.shape
    if gate_up_weight.shape[0] != 2 * I:
        raise KernelError(f"gemm_gated: weight {tuple(gate_up_weight.shape)} for {I} outputs")
    if out.dtype == torch.bfloat16:
        if _set_gated is None:
            _set_gated = _lib().ferris_gemm_set_gated_activation
            _set_gated.argtypes = [_I, _F]
            _set_gated.restype = None
        code = GATED_ACTIVATIONS[kind]
        try:  # the product that is launched next takes the activation; whatever happens, none is left behind
            if T <= 16 and gemm_skinny_enabled() and _skinny_takes(x, gate_up_weight, out, 2):
                _set_gated(code, float(limit))
                gemm_skinny(x, gate_up_weight, None, out, 3, up_row_offset=I)
                return
            if isinstance(x, LazyRMSNorm):
                x = x.materialize()
            if tensor_core_gemm_takes(x, gate_up_weight) and _lib().ferris_gemm_tcgen05_fuses_gated_activation(
                    _c_int(T), _c_int(I), _c_int(x.shape[1]), _c_int(out.stride(0)), _ptr(out)):
                _set_gated(code, float(limit))
                gemm_tcgen05(x, gate_up_weight, None, out, 3, up_row_offset=I)
                return
        finally:
            _set_gated(0, 0.0)
    if workspace is not None:
        gate_up = workspace.get("ffn_gate_up", (T, 2 * I), out.dtype)
    else:
        gate_up = torch.empty(T, 2 * I, dtype=out.dtype, device=out.device)
    gemm(x, gate_up_weight, None, gate_up)
    gated_activation(gate_up, out, kind, limit)


def gate_mul(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, kind: str = "sigmoid", scale: float = 1.0):
    """out = x * a(gate) * scale element by element, a = sigmoid or SiLU; fp32 arithmetic; ``out`` may be ``x``."""
    T, n, ldx = _rows(x, "gated rows")
    T2, n2, ldg = _rows(gate, "gate")
    T3, n3, ldo = _rows(out, "gated output")
    if (T2, n2) != (T, n) or (T3, n3) != (T, n) or gate.dtype != x.dtype or out.dtype != x.dtype or kind not in ("sigmoid", "silu"):
        raise KernelError(f"gate '{kind}': x {tuple(x.shape)}, gate {tuple(gate.shape)}, out {tuple(out.shape)}")
    _check(_lib().ferris_gate_mul(_ptr(x), _c_int(ldx), _ptr(gate), _c_int(ldg), _ptr(out), _c_int(ldo), _c_int(_dt(x, "gate")),
                                  _c_int(T), _c_int(n), _c_int(1 if kind == "silu" else 0), _c_float(scale), _stream()), "gate")


def scale_(x: torch.Tensor, scale: float):
    """x <- x * scale in place; fp32."""
    _need(x, "rows to scale", torch.float32)
    _check(_lib().ferris_scale(_ptr(x), ctypes.c_longlong(x.numel()), _c_float(scale), _stream()), "scale")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor):
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need(gate_up, "swiglu input")
    _need(out, "swiglu output", gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError(f"swiglu: input {tuple(gate_up.shape)}, output {tuple(out.shape)}")
    _check(_lib().ferris_swiglu(_ptr(gate_up), _ptr(out), _dt(out, "swiglu"), _c_int(T), _c_int(I), _stream()), "swiglu")


def rotary_angles(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor):
    """out [T, len(inv_freq), 2] fp32 = (cos, sin)(float(position) * inv_freq), as the rotary kernels form them."""
    _need(positions, "positions", torch.int32)
    _need(inv_freq, "rotary frequencies", torch.float32)
    _need(out, "rotary angles", torch.float32)
    T, half = positions.numel(), inv_freq.numel()
    if out.numel() != 2 * T * half:
        raise KernelError(f"rotary_angles: output {tuple(out.shape)} for {T} positions x {half} frequencies")
    _check(_lib().ferris_rotary_angles(_ptr(positions), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rotary angles")


QKV_ROPE_MIN_TOKENS = 128


def qkv_rope_gemm_takes(x, w, qkv, num_heads, num_kv_heads, head_dim, rotary_dim, k_cache) -> bool:
    """Whether ``qkv_rope_gemm`` takes this step: bf16 on the tensor cores, at least 128 tokens, heads of 64 or
    128 rotated whole."""
    return (isinstance(x, torch.Tensor) and qkv.shape[0] >= QKV_ROPE_MIN_TOKENS and head_dim in (64, 128)
            and rotary_dim == head_dim and qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and w.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim == qkv.shape[1]
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and tensor_core_gemm_takes(x, w))


def qkv_rope_gemm(x, w, bias, qkv, angles, slot_mapping, k_cache, v_cache, num_heads, num_kv_heads, head_dim):
    """The q/k/v product of a long step with rotation and cache write in its epilogue: ``qkv[:, :nh d]`` gets the
    rotated queries (its key and value columns are left as they were), the paged cache the rotated keys and
    the values at ``slot_mapping`` (None: nothing is stored, for a layer that reads another layer's cache).
    ``angles``: from ``rotary_angles`` for the step's positions."""
    T, K, ldx = _rows(x, "q/k/v input")
    rows_w, K2, ldw = _rows(w, "q/k/v weight")
    T2, N, ldo = _rows(qkv, "q/k/v output")
    _need(angles, "rotary angles", torch.float32)
    _need(k_cache, "key cache", torch.bfloat16)
    _need(v_cache, "value cache", torch.bfloat16)
    page_size = k_cache.shape[2]
    if (K != K2 or T != T2 or qkv.dtype != torch.bfloat16 or N != (num_heads + 2 * num_kv_heads) * head_dim
            or angles.numel() != T * head_dim or k_cache.dim() != 4
            or k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape):
        raise KernelError(f"qkv_rope_gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, qkv {tuple(qkv.shape)}, "
                          f"cache {tuple(k_cache.shape)}, angles {tuple(angles.shape)}")
    if bias is not None:
        _need(bias, "q/k/v bias", torch.float32)
        if bias.numel() != N:
            raise KernelError("qkv_rope_gemm: bias length differs from the output width")
    if slot_mapping is not None:
        _need(slot_mapping, "slot mapping", torch.int32)
        if slot_mapping.numel() != T:
            raise KernelError("qkv_rope_gemm: one cache slot per token is needed")
    _check(
        _lib().ferris_qkv_rope_gemm_tcgen05(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(),
                                            qkv.data_ptr(), T, K, ldx, ldw, ldo, rows_w, angles.data_ptr(),
                                            None if slot_mapping is None else slot_mapping.data_ptr(),
                                            k_cache.data_ptr(), v_cache.data_ptr(), num_heads, num_kv_heads, head_dim,
                                            page_size, _stream()),
        "q/k/v product with rotation",
    )


def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                     slot_mapping: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                     rotary_dim: int, page_size: int, write_kv: bool = True):
    """Rotate q and k of ``qkv`` [T, (nh + 2 nkv) d] by position; store k and v into the paged cache."""
    _need(qkv, "qkv")
    _need(positions, "positions", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or positions.numel() != T:
        raise KernelError(f"rope_cache_write: qkv {tuple(qkv.shape)} for {num_heads}+2x{num_kv_heads} heads of {head_dim}")
    if rotary_dim > 0:
        _need(inv_freq, "rotary frequencies", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rope_cache_write: one frequency per rotated pair is needed")
    if write_kv:
        _need(slot_mapping, "slot mapping", torch.int32)
        _need(k_cache, "key cache", qkv.dtype)
        _need(v_cache, "value cache", qkv.dtype)
        if slot_mapping.numel() != T or k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) \
                or v_cache.shape != k_cache.shape:
            raise KernelError(f"rope_cache_write: cache {tuple(k_cache.shape)} does not fit "
                              f"[pages, {num_kv_heads}, {page_size}, {head_dim}]")
    _check(
        _lib().ferris_rope_cache_write(_ptr(qkv), _dt(qkv, "qkv"), _ptr(positions), _ptr(inv_freq),
                                       _ptr(slot_mapping if write_kv else None), _ptr(k_cache if write_kv else None),
                                       _ptr(v_cache if write_kv else None), _c_int(T), _c_int(num_heads),
                                       _c_int(num_kv_heads), _c_int(head_dim), _c_int(rotary_dim), _c_int(page_size),
                                       _c_int(1 if write_kv else 0), _stream()),
        "rope_cache_write",
    )


_attention_tiled = True
ATTENTION_MAX_SHARES = 16  # most shares that the keys of a single token are cut into


class ScoreTerms:
    """What else enters an attention score and its softmax, per query head (fp32 [num_heads] tensors on the device, or
    None): ``slopes`` (the score of the key at j for the query at P gets slopes[h] * (j - P) added), ``log_r1`` and
    ``log_r2`` (it loses log_r1[h] * ln(1 + log_r2[h] * (P - j))), ``sink`` (the softmax's denominator also holds
    exp(sink[h]): a weight with no key and no value)."""

    __slots__ = ("slopes", "log_r1", "log_r2", "sink")

    def __init__(self, slopes=None, log_r1=None, log_r2=None, sink=None):
        self.slopes, self.log_r1, self.log_r2, self.sink = slopes, log_r1, log_r2, sink

    def any(self) -> bool:
        return any(t is not None for t in (self.slopes, self.log_r1, self.log_r2, self.sink))


def set_attention_tiled(on: bool = True) -> None:
    """Portions of prompts on the general attention's tiled kernel (True, the default) or on the kernel of single
    tokens (False), for comparisons."""
    global _attention_tiled
    _attention_tiled = bool(on)


def paged_attention_simt(qkv: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         block_tables: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor,
                         num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                         score_slopes=None, v_head_dim: Optional[int] = None,
                         max_q_len: int = 1, max_kv_len: int = 0, workspace=None, values_in_keys: bool = False,
                         chunk: int = 0):
    """General attention over the paged cache; q is read from the first nh*d columns of ``qkv``.
    ``window``: the query at position P sees the keys P - window + 1 .. P (0: all).  ``chunk`` (instead of a window):
    positions are counted off in chunks of that many from 0, and a query sees the keys of its own chunk up to itself.
    ``score_slopes`` (fp32 [num_heads]): the score of a query at position P and the key at position j gets
    slopes[head] * (j - P) added; or a ``ScoreTerms`` (slopes, a logarithmic distance penalty, a sink in the softmax's
    denominator).  ``v_head_dim``: size of a value head where it differs from the keys'.  ``values_in_keys``: a key's
    first ``v_head_dim`` elements are its value (``v_cache`` is then not read and may be None).
    ``max_q_len``: the most tokens a request brings; above one (portions of prompts) the kernel that shares tiles of
    keys among 64 query rows runs where it takes the geometry.  ``max_kv_len`` and ``workspace`` (a step of single
    tokens): the most keys a request holds, and where scratch comes from; the keys of a token are then cut into
    shares that run side by side, and query heads of one kv head share its keys."""
    dv = int(v_head_dim or head_dim)
    if chunk:
        if window or chunk < 0:
            raise KernelError(f"attention: a chunk of {chunk} and a window of {window} at once")
        window = chunk  # both bound the keys of a token; the kernels take a chunk as a negative window
    T, _, ldq = _rows(qkv, "attention queries")
    T2, width, ldo = _rows(out, "attention output")
    _need(k_cache, "key cache", qkv.dtype)
    v_stride = 0
    if values_in_keys:
        if dv > head_dim:
            raise KernelError(f"attention: keys of {head_dim} hold no values of {dv}")
        v_cache, v_stride = k_cache[..., :dv], head_dim
    else:
        _need(v_cache, "value cache", qkv.dtype)
    _need(block_tables, "block tables", torch.int32)
    _need(token_seq, "token-to-request map", torch.int32)
    _need(positions, "positions", torch.int32)
    terms = score_slopes if isinstance(score_slopes, ScoreTerms) else ScoreTerms(slopes=score_slopes)
    score_slopes = terms.slopes
    for name, t_ in (("logarithmic penalty", terms.log_r1), ("logarithmic penalty", terms.log_r2), ("sinks", terms.sink)):
        if t_ is not None:
            _need(t_, name, torch.float32)
            if t_.numel() != num_heads:
                raise KernelError(f"attention: one number of the {name} per query head is needed")
    if T != T2 or width != num_heads * dv or out.dtype != qkv.dtype or qkv.shape[1] < num_heads * head_dim:
        raise KernelError(f"attention: q {tuple(qkv.shape)}, out {tuple(out.shape)}")
    if (k_cache.dim() != 4 or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or block_tables.dim() != 2
            or v_cache.shape != (*k_cache.shape[:3], dv)):
        raise KernelError(f"attention: caches {tuple(k_cache.shape)} {tuple(v_cache.shape)}, tables {tuple(block_tables.shape)}")
    if score_slopes is not None:
        _need(score_slopes, "score slopes", torch.float32)
        if score_slopes.numel() != num_heads:
            raise KernelError("attention: one score slope per query head is needed")
    fn = _lib().ferris_paged_attention_simt
    extra = (_c_int(0), _ptr(None), ctypes.c_longlong(0))
    if max_q_len <= 1 and max_kv_len > 0 and workspace is not None:
        span = min(max_kv_len, window) if window else max_kv_len
        floats = T * num_heads * ATTENTION_MAX_SHARES * (dv + 2)
        scratch = workspace.get("attn_shares", (floats,), torch.float32)
        extra = (_c_int(span), _ptr(scratch), ctypes.c_longlong(floats))
    if max_q_len > 1 and _attention_tiled and (ldq * qkv.element_size()) % 16 == 0 and qkv.data_ptr() % 16 == 0 \
            and _lib().ferris_paged_attention_tiled_takes(_c_int(_dt(qkv, "attention")), _c_int(num_heads),
                                                          _c_int(num_kv_heads), _c_int(head_dim), _c_int(dv)):
        fn = _lib().ferris_paged_attention_tiled
        extra = ()
    _check(
        fn(_ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
                                           _dt(qkv, "attention"), _ptr(block_tables), _c_int(block_tables.shape[1]),
                                           _ptr(token_seq), _ptr(positions), _c_int(T), _c_int(num_heads),
                                           _c_int(num_kv_heads), _c_int(head_dim), _c_int(dv), _c_int(k_cache.shape[2]),
                                           _c_int(-chunk if chunk else (window or 0)), _c_float(scale), _ptr(score_slopes),
                                           _ptr(terms.log_r1),
                                           _ptr(terms.log_r2), _ptr(terms.sink), _c_int(v_stride), *extra, _stream()),
        "paged attention", 2 if extra and extra[0].value > 0 else 1,
    )


def embed_sinusoid(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, scale: float,
                   out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out[t, :] = table[ids[t], :] * scale + pe(positions[t]) as fp32, pe[2i] = sin(pos * freq[i]), pe[2i + 1] = cos(same)."""
    _need(table, "embedding table")
    _need(ids, "token ids", torch.int32)
    _need(positions, "positions", torch.int32)
    if freq is not None:  # None: no position vector, the scaled table row alone
        _need(freq, "position frequencies", torch.float32)
    _need(out, "embedding output", torch.float32)
    T, H = out.shape
    if (table.dim() != 2 or table.shape[1] != H or ids.numel() != T or positions.numel() != T
            or (freq is not None and freq.numel() != (H + 1) // 2)):
        raise KernelError(f"embed_sinusoid: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}, "
                          f"{0 if freq is None else freq.numel()} frequencies")
    _check(
        _lib().ferris_embed_sinusoid(_ptr(table), _c_int(_dt(table, "embedding table")), _ptr(ids), _ptr(positions),
                                     _ptr(freq), _c_float(scale), _ptr(out), _c_int(T), _c_int(H), _c_int(table.shape[0]),
                                     _ptr(status), _stream()),
        "embed_sinusoid",
    )


def grouped_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, out: torch.Tensor,
                    row_index: Optional[torch.Tensor] = None):
    """RMSNorm in ``groups`` equal consecutive parts of each row, each with a root mean square of its own; then the
    whole times ``weight``.  One group: the plain kernel."""
    if groups == 1:
        return rmsnorm(x, weight, eps, out, row_index)
    _need(x, "rmsnorm input", torch.float32)
    _need(weight, "rmsnorm weight", torch.float32)
    _need(out, "rmsnorm output")
    rows, H = out.shape
    if x.shape[1] != H or weight.numel() != H or groups < 1 or H % groups:
        raise KernelError(f"grouped rmsnorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, {groups} groups")
    if row_index is not None:
        _need(row_index, "rmsnorm row index", torch.int32)
        if row_index.numel() != rows:
            raise KernelError("rmsnorm: one row index per output row is needed")
    elif x.shape[0] != rows:
        raise KernelError("rmsnorm: input and output row counts differ")
    _check(
        _lib().ferris_grouped_rmsnorm(_ptr(x), _ptr(weight), _ptr(row_index), _ptr(out), _c_int(_dt(out, "rmsnorm output")),
                                      _c_int(rows), _c_int(H), _c_int(groups), _c_float(eps), _stream()),
        "grouped rmsnorm",
    )


def grouped_rmsnorm_pair(x: torch.Tensor, weight1: torch.Tensor, weight2: torch.Tensor, eps: float, groups: int,
                         out1: torch.Tensor, out2: torch.Tensor):
    """Two grouped RMSNorms of the same rows, with weights and outputs of their own, in one launch."""
    _need(x, "rmsnorm input", torch.float32)
    _need(weight1, "rmsnorm weight", torch.float32)
    _need(weight2, "rmsnorm weight", torch.float32)
    _need(out1, "rmsnorm output")
    _need(out2, "rmsnorm output", out1.dtype)
    rows, H = out1.shape
    if (x.shape != (rows, H) or out2.shape != (rows, H) or weight1.numel() != H or weight2.numel() != H or groups < 1
            or H % groups):
        raise KernelError(f"grouped rmsnorm pair: x {tuple(x.shape)}, outputs {tuple(out1.shape)} {tuple(out2.shape)}, "
                          f"{groups} groups")
    _check(
        _lib().ferris_grouped_rmsnorm_pair(_ptr(x), _ptr(weight1), _ptr(weight2), _ptr(out1), _ptr(out2),
                                           _c_int(_dt(out1, "rmsnorm output")), _c_int(rows), _c_int(H), _c_int(groups),
                                           _c_float(eps), _stream()),
        "grouped rmsnorm pair",
    )


def add_(h: torch.Tensor, x: torch.Tensor):
    """h += x, both fp32 and of one shape."""
    _need(h, "sum", torch.float32)
    _need(x, "addend", torch.float32)
    if h.shape != x.shape:
        raise KernelError(f"add: {tuple(h.shape)} += {tuple(x.shape)}")
    _check(_lib().ferris_add_f32(_ptr(h), _ptr(x), ctypes.c_longlong(h.numel()), _stream()), "add")


ACTIVATIONS = {"xielu": 0, "silu": 1, "relu2": 2}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str, params: Optional[torch.Tensor] = None):
    """out = a(x) element by element (``out`` may be ``x``).  ``xielu``: with softplus of the two numbers of
    ``params`` (fp32 [2]) as a = softplus(p), b = 1/2 + softplus(q): a z^2 + z / 2 for z > 0, b (exp(z) - 1 - z) + z / 2
    otherwise.  ``silu``: z sigmoid(z).  ``relu2``: max(z, 0)^2."""
    _need(x, "activation input")
    _need(out, "activation output", x.dtype)
    if kind not in ACTIVATIONS or out.shape != x.shape:
        raise KernelError(f"activation '{kind}': {tuple(x.shape)} -> {tuple(out.shape)}")
    if params is not None:
        _need(params, "activation parameters", torch.float32)
    if kind == "xielu" and (params is None or params.numel() != 2):
        raise KernelError("activation xielu: two numbers are needed")
    _check(_lib().ferris_activation(_ptr(x), _ptr(out), _c_int(_dt(x, "activation")), ctypes.c_longlong(x.numel()),
                                    _c_int(ACTIVATIONS[kind]), _ptr(params), _stream()), "activation")


def qk_prepare_cache_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                           k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], num_heads: int,
                           num_kv_heads: int, head_dim: int, v_head_dim: int, unit_norm_eps: Optional[float],
                           temperature: Optional[tuple], write_kv: bool = True):
    """Between the q/k/v product and attention where nothing rotates: q and k heads divided by their root mean
    square (``unit_norm_eps`` not None), q times 1 + coef * ln(floor((pos + 1) / every) + 1) (``temperature`` =
    (coef, every)), k and v into the paged cache.  ``qkv`` rows are [nh d | nkv d | nkv dv]; q is rewritten in place."""
    T, width, ld = _rows(qkv, "qkv")
    _need(positions, "positions", torch.int32)
    if width != (num_heads + num_kv_heads) * head_dim + num_kv_heads * v_head_dim or positions.numel() != T:
        raise KernelError(f"qk_prepare: qkv {tuple(qkv.shape)} for {num_heads}+{num_kv_heads} heads of {head_dim} and "
                          f"{num_kv_heads} of {v_head_dim}")
    page_size = 1
    if write_kv:
        _need(slot_mapping, "slot mapping", torch.int32)
        _need(k_cache, "key cache", qkv.dtype)
        _need(v_cache, "value cache", qkv.dtype)
        page_size = k_cache.shape[2]
        if (slot_mapping.numel() != T or k_cache.shape[1:] != (num_kv_heads, page_size, head_dim)
                or v_cache.shape != (*k_cache.shape[:3], v_head_dim)):
            raise KernelError(f"qk_prepare: caches {tuple(k_cache.shape)} {tuple(v_cache.shape)} do not fit")
    coef, every = temperature if temperature else (0.0, 0)
    _check(
        _lib().ferris_qk_prepare_cache_write(_ptr(qkv), _c_int(ld), _c_int(_dt(qkv, "qkv")), _ptr(positions),
                                             _ptr(slot_mapping if write_kv else None), _ptr(k_cache if write_kv else None),
                                             _ptr(v_cache if write_kv else None), _c_int(T), _c_int(num_heads),
                                             _c_int(num_kv_heads), _c_int(head_dim), _c_int(v_head_dim), _c_int(page_size),
                                             _c_int(0 if unit_norm_eps is None else 1), _c_float(unit_norm_eps or 0.0),
                                             _c_float(coef), _c_int(int(every)), _c_int(1 if write_kv else 0), _stream()),
        "qk_prepare_cache_write",
    )


def short_conv(y: torch.Tensor, out: torch.Tensor, weight: torch.Tensor, state: Optional[torch.Tensor], ctx,
               advance: bool = True, bias: Optional[torch.Tensor] = None, residual: bool = True, silu: bool = False):
    """out = y + causal convolution of y over time on each channel (``weight`` fp32 [channels, taps]; without
    ``residual`` the convolution alone; ``bias`` fp32 [channels] added; ``silu``: SiLU of the sum), a request's
    ``taps - 1`` inputs before the step taken from ``state`` (fp32 [slots, taps - 1, channels]) and, with
    ``advance``, the state moved on to the step's end.  ``ctx``: the step context (device arrays only)."""
    T, C, ldy = _rows(y, "convolution input")
    T2, C2, ldo = _rows(out, "convolution output")
    _need(weight, "convolution weight", torch.float32)
    taps = weight.shape[1]
    if (T2, C2) != (T, C) or out.dtype != y.dtype or weight.shape != (C, taps) or y.data_ptr() == out.data_ptr():
        raise KernelError(f"short conv: y {tuple(y.shape)}, out {tuple(out.shape)}, weight {tuple(weight.shape)}")
    if bias is not None:
        _need(bias, "convolution bias", torch.float32)
        if bias.numel() != C:
            raise KernelError(f"short conv: {bias.numel()} biases for {C} channels")
    if taps > 1:
        _need(state, "convolution state", torch.float32)
        if state.shape[1:] != (taps - 1, C):
            raise KernelError(f"short conv: state {tuple(state.shape)} for {taps} taps of {C} channels")
    single = bool(advance and getattr(ctx, "max_q_len", 0) == 1 and T == ctx.num_seqs)  # one token each: one launch
    kernels = 2 if (advance and taps > 1 and not single) else 1
    _check(
        _lib().ferris_short_conv(_ptr(y), _c_int(ldy), _ptr(out), _c_int(ldo), _c_int(_dt(y, "short conv")), _ptr(weight),
                                 _ptr(state if taps > 1 else None), _ptr(ctx.token_seq), _ptr(ctx.positions),
                                 _ptr(ctx.seq_q_start), _ptr(ctx.seq_start_pos), _ptr(ctx.seq_state_slot), _c_int(T),
                                 _c_int(ctx.num_seqs), _c_int(C), _c_int(taps), _c_int(1 if advance else 0),
                                 _c_int(1 if single else 0), _ptr(bias), _c_int(1 if residual else 0),
                                 _c_int(1 if silu else 0), _stream()),
        "short conv", kernels,
    )


LINEAR_ATTENTION_SEGMENT = 128


def linear_attention(qkv: torch.Tensor, offsets: tuple, out: torch.Tensor, state: torch.Tensor, decay: torch.Tensor,
                     ctx, heads: int, dim: int, vdim: int, silu: bool = False, write_state: bool = True,
                     segment: Optional[int] = None, rotary: Optional["RotaryTable"] = None, k_scale: float = 1.0):
    """Decayed linear attention of the step's tokens, request by request from each request's state:
    S <- decay[h] S + k v^T, o = S^T q per head.  ``qkv`` rows hold q, k heads (heads x dim) and v heads
    (heads x vdim) at the column ``offsets`` (q, k, v); ``out`` fp32 [T, heads x vdim]; ``state`` fp32
    [slots, heads, vdim, dim].  ``silu``: q, k and v pass through SiLU on the way in.  A request that brings more
    than ``segment`` tokens (128 by default) runs as segments side by side: a pass that sums each segment alone, one
    that carries the state from segment to segment, one that forms the outputs (scratch from the step's workspace).
    ``rotary``: q and k are rotated by the tokens' positions (``ctx.positions``) on their way in; ``k_scale``: k is then
    multiplied by it.  Both in fp32, so what enters the recurrence is never rounded."""
    T, width, ld = _rows(qkv, "linear attention input")
    T2, n, ldo = _rows(out, "linear attention output")
    _need(state, "linear attention state", torch.float32)
    _need(decay, "decays", torch.float32)
    q_off, k_off, v_off = (int(o) for o in offsets)
    if (T2 != T or out.dtype != torch.float32 or n != heads * vdim or state.shape[1:] != (heads, vdim, dim)
            or decay.numel() != heads or max(q_off, k_off) + heads * dim > width or v_off + heads * vdim > width):
        raise KernelError(f"linear attention: qkv {tuple(qkv.shape)}, out {tuple(out.shape)}, state {tuple(state.shape)}")
    seg = int(segment or LINEAR_ATTENTION_SEGMENT)
    longest = int(getattr(ctx, "max_q_len", 0) or T)
    segs_max = max(1, -(-longest // seg))
    scratch = None
    if segs_max > 1:
        floats = (T // seg + ctx.num_seqs + 1) * heads * vdim * dim
        ws = getattr(ctx, "workspace", None)
        scratch = ws.get("linear_attn_segments", (floats,), torch.float32) if ws is not None else \
            torch.empty(floats, dtype=torch.float32, device=qkv.device)
    _check(
        _lib().ferris_linear_attention(_ptr(qkv), _c_int(ld), _c_int(q_off), _c_int(k_off), _c_int(v_off),
                                       _c_int(_dt(qkv, "linear attention")), _ptr(out), _c_int(ldo), _ptr(state),
                                       _ptr(decay), _ptr(ctx.seq_q_start), _ptr(ctx.seq_state_slot), _c_int(ctx.num_seqs),
                                       _c_int(heads), _c_int(dim), _c_int(vdim), _c_int(1 if silu else 0),
                                       _c_int(1 if write_state else 0), _c_int(seg), _c_int(segs_max), _ptr(scratch),
                                       *_rotary_args(rotary, ctx, dim, qkv.device), _c_float(k_scale), _stream()),
        "linear attention", 1 if segs_max == 1 else 3,
    )


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor):
    """out = rmsnorm(o) * weight * sigmoid(gate), row by row; o fp32, gate and out in the activations' type."""
    T, n, ldi = _rows(o, "gated norm input")
    T2, n2, ldg = _rows(gate, "gate")
    T3, n3, ldo = _rows(out, "gated norm output")
    _need(weight, "gated norm weight", torch.float32)
    if (o.dtype != torch.float32 or (T2, n2) != (T, n) or (T3, n3) != (T, n) or gate.dtype != out.dtype
            or weight.numel() != n):
        raise KernelError(f"gated rmsnorm: o {tuple(o.shape)}, gate {tuple(gate.shape)}, out {tuple(out.shape)}")
    _check(
        _lib().ferris_gated_rmsnorm(_ptr(o), _c_int(ldi), _ptr(gate), _c_int(ldg), _ptr(weight), _ptr(out), _c_int(ldo),
                                    _c_int(_dt(out, "gated norm")), _c_int(T), _c_int(n), _c_float(eps), _stream()),
        "gated rmsnorm",
    )


def recurrence_gates(proj: torch.Tensor, a_off: int, b_off: Optional[int], A_log: torch.Tensor, dt_bias: torch.Tensor,
                     decay: torch.Tensor, beta: torch.Tensor, heads: int, unit_norm: Optional[tuple] = None):
    """Per token and head: decay = exp(-exp(A_log) * dt) with dt = softplus(proj[:, a_off + h] + dt_bias); beta =
    sigmoid(proj[:, b_off + h]), or dt itself where ``b_off`` is None.  ``unit_norm`` = (rows, q_off, k_off, qk_heads,
    dim, eps, q_mul, qscale, kscale): the factors that make the q and k heads of ``rows`` unit vectors
    (1 / sqrt(sum x^2 + eps); q's also times q_mul), fp32 [T, qk_heads] each.  All in fp32."""
    T, width, ld = _rows(proj, "recurrence gates input")
    _need(A_log, "A_log", torch.float32)
    _need(dt_bias, "dt_bias", torch.float32)
    _need(decay, "decays", torch.float32)
    _need(beta, "step sizes", torch.float32)
    if (A_log.numel() != heads or dt_bias.numel() != heads or decay.shape != (T, heads) or beta.shape != (T, heads)
            or a_off + heads > width or (b_off is not None and b_off + heads > width)):
        raise KernelError(f"recurrence gates: proj {tuple(proj.shape)}, {heads} heads, decay {tuple(decay.shape)}")
    qk, ldqk, q_off, k_off, qk_heads, dim, eps, q_mul, qscale, kscale = None, 0, 0, 0, 0, 0, 0.0, 1.0, None, None
    if unit_norm is not None:
        qk, q_off, k_off, qk_heads, dim, eps, q_mul, qscale, kscale = unit_norm
        T2, w2, ldqk = _rows(qk, "recurrence q and k")
        _need(qscale, "q factors", torch.float32)
        _need(kscale, "k factors", torch.float32)
        if (T2 != T or qk.dtype != proj.dtype or max(q_off, k_off) + qk_heads * dim > w2 or qscale.shape != (T, qk_heads)
                or kscale.shape != (T, qk_heads)):
            raise KernelError(f"recurrence gates: q/k rows {tuple(qk.shape)} for {qk_heads} heads of {dim}")
    _check(
        _lib().ferris_recurrence_gates(_ptr(proj), _c_int(ld), _c_int(_dt(proj, "recurrence gates")), _c_int(a_off),
                                       _c_int(-1 if b_off is None else b_off), _ptr(A_log), _ptr(dt_bias), _ptr(decay),
                                       _ptr(beta), _c_int(1 if b_off is None else 0), _ptr(qk), _c_int(ldqk), _c_int(q_off),
                                       _c_int(k_off), _c_int(qk_heads), _c_int(dim), _c_float(eps), _c_float(q_mul),
                                       _ptr(qscale), _ptr(kscale), _c_int(T), _c_int(heads), _stream()),
        "recurrence gates",
    )


def gated_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor,
                     out: torch.Tensor, state: torch.Tensor, ctx, heads: int, qk_heads: int, dim: int, vdim: int,
                     delta_rule: bool, qscale: Optional[torch.Tensor] = None, kscale: Optional[torch.Tensor] = None,
                     skip: Optional[torch.Tensor] = None, write_state: bool = True):
    """The recurrence of the step's tokens, request by request from each request's state (fp32 [slots, heads, vdim, dim]: S transposed):
    plain: S <- decay S + k (beta v)^T, o = S^T q + skip v;  delta rule: S <- decay S, u = beta (v - S^T k), S <- S + k u^T,
    o = S^T q.  ``q``, ``k``: [T, qk_heads x dim] (views with contiguous rows; value head h uses q/k head
    h / (heads / qk_heads)), optionally times one fp32 factor per (token, q/k head) each; ``v``: [T, heads x vdim];
    ``decay``, ``beta``: fp32 [T, heads]; ``out``: fp32 [T, heads x vdim]."""
    T, wq, ldq = _rows(q, "recurrence queries")
    T1, wk, ldk = _rows(k, "recurrence keys")
    T2, wv, ldv = _rows(v, "recurrence values")
    T3, wo, ldo = _rows(out, "recurrence output")
    _need(state, "recurrence state", torch.float32)
    _need(decay, "decays", torch.float32)
    _need(beta, "step sizes", torch.float32)
    if (not (T == T1 == T2 == T3) or wq != qk_heads * dim or wk != qk_heads * dim or wv != heads * vdim or wo != heads * vdim
            or out.dtype != torch.float32 or k.dtype != q.dtype or v.dtype != q.dtype or state.shape[1:] != (heads, vdim, dim)
            or decay.shape != (T, heads) or beta.shape != (T, heads)):
        raise KernelError(f"recurrence: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}, out {tuple(out.shape)}, "
                          f"state {tuple(state.shape)}")
    for name, t_ in (("q factors", qscale), ("k factors", kscale)):
        if t_ is not None:
            _need(t_, name, torch.float32)
            if t_.shape != (T, qk_heads):
                raise KernelError(f"recurrence: {name} {tuple(t_.shape)}")
    if skip is not None:
        _need(skip, "skip weights", torch.float32)
        if skip.numel() != heads:
            raise KernelError("recurrence: one skip weight per head is needed")
    _check(
        _lib().ferris_gated_recurrence(_ptr(q), _c_int(ldq), _ptr(k), _c_int(ldk), _ptr(v), _c_int(ldv),
                                       _c_int(_dt(q, "recurrence")), _ptr(decay), _ptr(beta), _ptr(qscale), _ptr(kscale),
                                       _ptr(skip), _ptr(out), _c_int(ldo), _ptr(state), _ptr(ctx.seq_q_start),
                                       _ptr(ctx.seq_state_slot), _c_int(ctx.num_seqs), _c_int(heads), _c_int(qk_heads),
                                       _c_int(dim), _c_int(vdim), _c_int(1 if delta_rule else 0),
                                       _c_int(1 if write_state else 0), _c_int(int(getattr(ctx, "max_q_len", 0) or T)),
                                       _stream()),
        "gated recurrence",
    )


def gated_group_norm(o: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                     group: int, gate_kind: str = "sigmoid", gate_first: bool = False):
    """out = norm(o [* a(gate)]) * weight [* a(gate)]: every ``group`` consecutive columns divided by their own
    sqrt(mean(.^2) + eps); ``weight`` (fp32) repeats every ``weight.numel()`` columns; the gate (a = "sigmoid" or
    "silu") multiplies before the norm (``gate_first``) or after it.  o fp32; gate and out in the activations' type."""
    T, n, ldi = _rows(o, "gated norm input")
    T3, n3, ldo = _rows(out, "gated norm output")
    _need(weight, "gated norm weight", torch.float32)
    ldg = 0
    if gate is not None:
        T2, n2, ldg = _rows(gate, "gate")
        if (T2, n2) != (T, n) or gate.dtype != out.dtype:
            raise KernelError(f"gated group norm: gate {tuple(gate.shape)} for {tuple(o.shape)}")
    if o.dtype != torch.float32 or (T3, n3) != (T, n) or group <= 0 or n % group or n % weight.numel() \
            or gate_kind not in ("sigmoid", "silu"):
        raise KernelError(f"gated group norm: o {tuple(o.shape)}, out {tuple(out.shape)}, groups of {group}, "
                          f"{weight.numel()} weights, gate '{gate_kind}'")
    _check(
        _lib().ferris_gated_group_norm(_ptr(o), _c_int(ldi), _ptr(gate), _c_int(ldg), _ptr(weight), _c_int(weight.numel()),
                                       _ptr(out), _c_int(ldo), _c_int(_dt(out, "gated norm")), _c_int(T), _c_int(n),
                                       _c_int(group), _c_float(eps), _c_int(1 if gate_kind == "silu" else 0),
                                       _c_int(1 if gate_first else 0), _stream()),
        "gated group norm",
    )


ROW_DECAY_SEGMENT = 128  # tokens of a segment where a long portion runs as segments side by side
ROW_DECAY_SEGMENTS_FROM = 384  # the longest request of a step from which on that pays


def row_decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, row_z: torch.Tensor, power: float,
                         out: torch.Tensor, state: torch.Tensor, ctx, num_heads: int, head_dim: int, v_head_dim: int,
                         q_scale: float = 1.0, write_state: bool = True, segment: Optional[int] = None):
    """Linear attention with a decay per key channel that changes with every token: per head
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = q_scale S_t^T q_t, alpha_t = sigmoid(row_z[t])^power (fp32, formed in
    the kernel).  q, k: [T, heads x dim], v: [T, heads x vdim] (views with contiguous rows); row_z fp32 [T, heads x dim];
    out fp32 [T, heads x vdim]; state fp32 [slots, heads, vdim, dim] (transposed), carried in the requests' slots.
    A step whose longest request brings ROW_DECAY_SEGMENTS_FROM tokens or more (or any step, with ``segment`` given)
    runs as segments of ``segment`` tokens side by side: a pass that sums each segment alone, one that multiplies up
    its rows' decays, one that carries the state from segment to segment, one that forms the outputs."""
    T, wq, ldq = _rows(q, "recurrence q")
    _, wk, ldk = _rows(k, "recurrence k")
    _, wv, ldv = _rows(v, "recurrence v")
    _, wz, ldz = _rows(row_z, "recurrence decays")
    _, wo, ldo = _rows(out, "recurrence output")
    _need(state, "recurrent state", torch.float32)
    if (wq != num_heads * head_dim or wk != wq or wz != wq or wv != num_heads * v_head_dim or wo != wv
            or row_z.dtype != torch.float32 or out.dtype != torch.float32 or k.dtype != q.dtype or v.dtype != q.dtype
            or state.shape[1:] != (num_heads, v_head_dim, head_dim)):
        raise KernelError(f"row-decay recurrence: q {tuple(q.shape)}, v {tuple(v.shape)}, decays {tuple(row_z.shape)}, "
                          f"state {tuple(state.shape)}")
    longest = int(getattr(ctx, "max_q_len", 0) or T)
    seg = int(segment or ROW_DECAY_SEGMENT)
    segs_max = max(1, -(-longest // seg)) if (segment is not None or longest >= ROW_DECAY_SEGMENTS_FROM) else 1
    scratch_s = scratch_p = None
    if segs_max > 1:
        places = T // seg + ctx.num_seqs + 1
        ws = getattr(ctx, "workspace", None)
        get = ws.get if ws is not None else (lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=q.device))
        scratch_s = get("row_decay_segments", (places * num_heads * v_head_dim * head_dim,), torch.float32)
        scratch_p = get("row_decay_products", (places * num_heads * head_dim,), torch.float32)
    _check(
        _lib().ferris_row_decay_recurrence(_ptr(q), _c_int(ldq), _ptr(k), _c_int(ldk), _ptr(v), _c_int(ldv),
                                           _c_int(_dt(q, "recurrence")), _ptr(row_z), _c_int(ldz), _c_float(power),
                                           _c_float(q_scale), _ptr(out), _c_int(ldo), _ptr(state), _ptr(ctx.seq_q_start),
                                           _ptr(ctx.seq_state_slot), _c_int(ctx.num_seqs), _c_int(num_heads),
                                           _c_int(head_dim), _c_int(v_head_dim), _c_int(1 if write_state else 0),
                                           _c_int(longest), _c_int(seg), _c_int(segs_max), _ptr(scratch_s), _ptr(scratch_p),
                                           _stream()),
        "row-decay recurrence", 1 if segs_max == 1 else 4,
    )


RGLRU_TENSOR_CORE_MIN_TOKENS = 256  # from here on a bf16 step forms the gates' products on the tensor cores (at 64 tokens the CUDA-core form takes 16 us, this one 22)


def rglru_gates(u: torch.Tensor, wa_t: torch.Tensor, wi_t: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor,
                softplus_lam: torch.Tensor, a_out: Optional[torch.Tensor], b_out: Optional[torch.Tensor], decay_factor: float,
                step: Optional[tuple] = None, stored: Optional[tuple] = None):
    """The gates of a gated linear recurrent unit: per block n of the channels r = sigmoid(Ra[n] u_n + ba),
    i = sigmoid(Ri[n] u_n + bi); log a = -decay_factor r softplus_lam; b = sqrt(1 - a^2) i u.  ``wa_t``, ``wi_t``:
    [blocks, in, out] (the matrices transposed) in u's type; ba, bi, softplus_lam fp32 [C]; a_out (which receives log a,
    not a: the scan never rounds a decay close to one to 24 bits) and b_out fp32 [T, C].
    ``step`` = (state fp32 [slots, C], ctx, y or None, out, gelu, write_state) for a step in which every request brings
    one token: the kernel moves the state on itself and writes out = s * act(y) (see ``rglru_scan``); a_out and b_out
    are then not needed.  ``stored`` = (Ra, Ri) as the folder stores them ([blocks, out, in]): a bf16 step of at least
    RGLRU_TENSOR_CORE_MIN_TOKENS tokens with gate blocks of a multiple of 64 channels then forms the two products on the
    tensor cores (bf16 operands, fp32 sums; the same epilogue)."""
    T, C, ldu = _rows(u, "recurrent unit input")
    _need(wa_t, "recurrence gate matrices", u.dtype)
    _need(wi_t, "input gate matrices", u.dtype)
    blocks = wa_t.shape[0]
    bs = C // max(blocks, 1)
    for t_, name in ((ba, "recurrence gate bias"), (bi, "input gate bias"), (softplus_lam, "decay rates")):
        _need(t_, name, torch.float32)
    if (stored is not None and step is None and u.dtype == torch.bfloat16 and T >= RGLRU_TENSOR_CORE_MIN_TOKENS
            and bs % 64 == 0 and ldu % 8 == 0 and u.data_ptr() % 32 == 0):
        wa, wi = stored
        _need(wa, "recurrence gate matrices", u.dtype)
        _need(wi, "input gate matrices", u.dtype)
        _need(a_out, "decays", torch.float32)
        _need(b_out, "gated inputs", torch.float32)
        if (wa.shape != (blocks, bs, bs) or wi.shape != wa.shape or ba.numel() != C or bi.numel() != C
                or softplus_lam.numel() != C or a_out.shape != (T, C) or b_out.shape != (T, C)):
            raise KernelError(f"recurrent unit gates: u {tuple(u.shape)}, matrices {tuple(wa.shape)}")
        _check(_lib().ferris_rglru_gates_mma(_ptr(u), _c_int(ldu), _ptr(wa), _ptr(wi), _ptr(ba), _ptr(bi), _ptr(softplus_lam),
                                             _ptr(a_out), _ptr(b_out), _c_int(T), _c_int(C), _c_int(blocks),
                                             _c_float(decay_factor), _stream()), "recurrent unit gates (tensor cores)")
        return
    state = slots = y = out = None
    ldy = ldo = 0
    gelu = write_state = False
    if step is not None:
        state, ctx, y, out, gelu, write_state = step
        _need(state, "recurrent state", torch.float32)
        _, Co, ldo = _rows(out, "recurrent unit output")
        if y is not None:
            _, Cy, ldy = _rows(y, "recurrent unit branch")
        if (T != ctx.num_seqs or state.dim() != 2 or state.shape[1] != C or out.shape != (T, C) or out.dtype != u.dtype
                or (y is not None and (y.shape != (T, C) or y.dtype != u.dtype))):
            raise KernelError(f"recurrent unit step: {T} rows of {ctx.num_seqs} requests, state {tuple(state.shape)}")
        slots = ctx.seq_state_slot
    else:
        _need(a_out, "decays", torch.float32)
        _need(b_out, "gated inputs", torch.float32)
        if a_out.shape != (T, C) or b_out.shape != (T, C):
            raise KernelError(f"recurrent unit gates: outputs {tuple(a_out.shape)}, {tuple(b_out.shape)} for {T} x {C}")
    if (wa_t.shape != (blocks, bs, bs) or wi_t.shape != wa_t.shape or blocks * bs != C or ba.numel() != C or bi.numel() != C
            or softplus_lam.numel() != C):
        raise KernelError(f"recurrent unit gates: u {tuple(u.shape)}, matrices {tuple(wa_t.shape)}")
    _check(_lib().ferris_rglru_gates(_ptr(u), _c_int(ldu), _c_int(_dt(u, "recurrent unit")), _ptr(wa_t), _ptr(wi_t), _ptr(ba),
                                     _ptr(bi), _ptr(softplus_lam), _ptr(a_out), _ptr(b_out), _c_int(T), _c_int(C),
                                     _c_int(blocks), _c_float(decay_factor), _ptr(state), _ptr(slots), _ptr(y), _c_int(ldy),
                                     _ptr(out), _c_int(ldo), _c_int(1 if gelu else 0), _c_int(1 if write_state else 0),
                                     _stream()), "recurrent unit gates")


def rglru_scan(a: torch.Tensor, b: torch.Tensor, y: Optional[torch.Tensor], out: torch.Tensor, state: torch.Tensor, ctx,
               gelu: bool = True, write_state: bool = True):
    """s_t = exp(a_t) s_(t-1) + b_t per (request, channel) from the request's slot of ``state`` (fp32 [slots, C]), formed as
    s + (expm1(a_t) s + b_t); out_t = s_t * act(y_t), act the tanh form of GELU (``gelu``) or nothing; without ``y`` the
    state itself.  a (the LOGARITHMS of the decays) and b fp32 [T, C]; y, out in the activations' type (views with
    contiguous rows)."""
    _need(a, "decays", torch.float32)
    _need(b, "gated inputs", torch.float32)
    _need(state, "recurrent state", torch.float32)
    T, C = a.shape
    T2, C2, ldo = _rows(out, "recurrent unit output")
    ldy = 0
    if y is not None:
        T3, C3, ldy = _rows(y, "recurrent unit branch")
        if (T3, C3) != (T, C) or y.dtype != out.dtype:
            raise KernelError(f"recurrent unit scan: branch {tuple(y.shape)} for {T} x {C}")
    if b.shape != (T, C) or (T2, C2) != (T, C) or state.dim() != 2 or state.shape[1] != C:
        raise KernelError(f"recurrent unit scan: a {tuple(a.shape)}, b {tuple(b.shape)}, out {tuple(out.shape)}, "
                          f"state {tuple(state.shape)}")
    single = bool(getattr(ctx, "max_q_len", 0) == 1 and T == ctx.num_seqs)
    _check(_lib().ferris_rglru_scan(_ptr(a), _ptr(b), _ptr(y), _c_int(ldy), _ptr(out), _c_int(ldo),
                                    _c_int(_dt(out, "recurrent unit")), _ptr(state), _ptr(ctx.seq_q_start),
                                    _ptr(ctx.seq_state_slot), _c_int(T), _c_int(ctx.num_seqs), _c_int(C),
                                    _c_int(1 if gelu else 0), _c_int(1 if write_state else 0), _c_int(1 if single else 0),
                                    _stream()), "recurrent unit scan")


def streams_expand(h: torch.Tensor, xs: torch.Tensor, streams: int):
    """xs [T, streams x W] = ``streams`` copies of every row of h [T, W]; both fp32."""
    _need(h, "residual rows", torch.float32)
    _need(xs, "residual streams", torch.float32)
    T, W = h.shape
    if xs.shape != (T, streams * W):
        raise KernelError(f"streams: {tuple(h.shape)} into {tuple(xs.shape)} as {streams} streams")
    _check(_lib().ferris_streams_expand(_ptr(h), _ptr(xs), _c_int(T), _c_int(streams), _c_int(W), _stream()), "streams expand")


def streams_sum(xs: torch.Tensor, h: torch.Tensor, streams: int):
    """h [T, W] = the sum of the ``streams`` rows of every token in xs [T, streams x W]; both fp32."""
    _need(h, "residual rows", torch.float32)
    _need(xs, "residual streams", torch.float32)
    T, W = h.shape
    if xs.shape != (T, streams * W):
        raise KernelError(f"streams: {tuple(xs.shape)} into {tuple(h.shape)} as {streams} streams")
    _check(_lib().ferris_streams_sum(_ptr(xs), _ptr(h), _c_int(T), _c_int(streams), _c_int(W), _stream()), "streams sum")


def streams_step(xs: torch.Tensor, streams: int, write: Optional[tuple] = None, read: Optional[tuple] = None,
                 shift: Optional[tuple] = None):
    """One pass over every token's residual streams (xs fp32 [T, streams x W]): ``write`` = (y fp32 [T, W], mix fp32
    [streams, streams] indexed [from, to], out fp32 [streams]): x_r <- sum_s mix[s, r] x_s + out[r] y, all r from the
    old streams; then ``read`` = (in fp32 [streams], norm weight fp32 [W], eps, out [T, W] in the activations' type):
    out = rmsnorm(sum_s in[s] x_s) * weight.  Either may be None.  ``shift`` = (weights fp32 [W], state fp32 [slots, W],
    ctx), only in a step where every request brings one token: the read's rows are token-shifted on their way out, as
    ``token_shift`` does, from and to the requests' states."""
    _need(xs, "residual streams", torch.float32)
    T = xs.shape[0]
    if xs.dim() != 2 or xs.shape[1] % streams:
        raise KernelError(f"streams: {tuple(xs.shape)} as {streams} streams")
    W = xs.shape[1] // streams
    y = mix = out_w = in_w = norm_w = out = None
    eps = 0.0
    if write is not None:
        y, mix, out_w = write
        _need(y, "sublayer result", torch.float32)
        _need(mix, "stream mixing matrix", torch.float32)
        _need(out_w, "stream output weights", torch.float32)
        if y.shape != (T, W) or mix.numel() != streams * streams or out_w.numel() != streams:
            raise KernelError(f"streams write: y {tuple(y.shape)}, mix {tuple(mix.shape)}, out {tuple(out_w.shape)}")
    if read is not None:
        in_w, norm_w, eps, out = read
        _need(in_w, "stream input weights", torch.float32)
        _need(norm_w, "norm weight", torch.float32)
        _need(out, "normed rows")
        if in_w.numel() != streams or norm_w.numel() != W or out.shape != (T, W):
            raise KernelError(f"streams read: in {tuple(in_w.shape)}, norm {tuple(norm_w.shape)}, out {tuple(out.shape)}")
    sw = sstate = spos = sslot = None
    if shift is not None:
        sw, sstate, ctx = shift
        _need(sw, "token shift weights", torch.float32)
        _need(sstate, "token shift state", torch.float32)
        if read is None or sw.numel() != W or sstate.dim() != 2 or sstate.shape[1] != W or ctx.max_q_len != 1 \
                or ctx.num_seqs != T:
            raise KernelError("streams step: a token shift goes with a read in a step of single tokens")
        spos, sslot = ctx.positions, ctx.seq_state_slot
    _check(
        _lib().ferris_streams_step(_ptr(xs), _ptr(y), _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(norm_w), _c_float(eps),
                                   _ptr(out), _c_int(_dt(out, "normed rows") if out is not None else F32), _c_int(T),
                                   _c_int(streams), _c_int(W), _ptr(sw), _ptr(sstate), _ptr(spos), _ptr(sslot), _stream()),
        "streams step",
    )


def token_shift(x: torch.Tensor, out: torch.Tensor, shift: torch.Tensor, state: torch.Tensor, ctx, advance: bool = True):
    """out_t = x_t + (x_(t-1) - x_t) * shift, x_(t-1) the unshifted row of the request's token before (zeros at position
    0; across steps from ``state``, fp32 [slots, W], which ``advance`` moves on to the request's last row of this step)."""
    _need(x, "token shift input")
    _need(out, "token shift output", x.dtype)
    _need(shift, "token shift weights", torch.float32)
    _need(state, "token shift state", torch.float32)
    T, W = x.shape
    if out.shape != (T, W) or shift.numel() != W or state.dim() != 2 or state.shape[1] != W or x.data_ptr() == out.data_ptr():
        raise KernelError(f"token shift: x {tuple(x.shape)}, out {tuple(out.shape)}, state {tuple(state.shape)}")
    single = bool(advance and getattr(ctx, "max_q_len", 0) == 1 and T == ctx.num_seqs)
    _check(
        _lib().ferris_token_shift(_ptr(x), _ptr(out), _c_int(_dt(x, "token shift")), _ptr(shift), _ptr(state),
                                  _ptr(ctx.token_seq), _ptr(ctx.positions), _ptr(ctx.seq_q_start), _ptr(ctx.seq_start_pos),
                                  _ptr(ctx.seq_state_slot), _c_int(T), _c_int(ctx.num_seqs), _c_int(W),
                                  _c_int(1 if advance else 0), _c_int(1 if single else 0), _stream()),
        "token shift", 2 if (advance and not single) else 1,
    )


def branch_norm_sum(h: torch.Tensor, branches: list, coef: float, eps: float, accumulate: bool = True):
    """h += coef * sum_b rmsnorm(y_b) * w_b over ``branches`` = [(y_b fp32 [T, W], w_b fp32 [W]), ...] (one to four);
    without ``accumulate`` the sum replaces what h held."""
    _need(h, "residual rows", torch.float32)
    n = len(branches)
    ys = (ctypes.c_void_p * n)()
    ws = (ctypes.c_void_p * n)()
    for i, (y, w) in enumerate(branches):
        _need(y, "branch result", torch.float32)
        _need(w, "branch norm weight", torch.float32)
        if y.shape != h.shape or w.numel() != h.shape[1]:
            raise KernelError(f"branch norm: y {tuple(y.shape)}, w {tuple(w.shape)} for h {tuple(h.shape)}")
        ys[i], ws[i] = y.data_ptr(), w.data_ptr()
    _check(_lib().ferris_branch_norm_sum(ys, ws, _c_int(n), _c_float(coef), _c_float(eps), _ptr(h), _c_int(h.shape[0]),
                                         _c_int(h.shape[1]), _c_int(1 if accumulate else 0), _stream()), "branch norm sum")


def latent_prepare(proj: torch.Tensor, q_off: int, dkv_off: int, norm_weight: torch.Tensor, eps: float,
                   positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dims: int,
                   slot_mapping: Optional[torch.Tensor], cache: Optional[torch.Tensor], q_att: torch.Tensor, heads: int,
                   dim: int, rot: int, rank: int, write_kv: bool = True):
    """Between the input product and attention over a shared latent.  ``proj`` rows hold ``heads`` x [dim plain | rot
    rotated] query dimensions from ``q_off`` and [rank latent | rot key] from ``dkv_off``.  The latent is RMS-normed
    with ``norm_weight``, the key part and the heads' rotated query parts are rotated (rotate-half over the first
    ``rot_dims``, angle = position * inv_freq[i]), [latent | key part] becomes the token's cache row (``cache``
    [pages, 1, page size, rank + rot]) and the rotated query parts go to ``q_att`` [T, heads x (rank + rot)], behind
    the first ``rank`` columns of each head (which the absorbed plain queries fill)."""
    T, width, ld = _rows(proj, "latent input")
    T2, wq, ldqa = _rows(q_att, "latent queries")
    _need(positions, "positions", torch.int32)
    if (T2 != T or q_att.dtype != proj.dtype or wq != heads * (rank + rot) or q_off + heads * (dim + rot) > width
            or dkv_off + rank + rot > width or positions.numel() != T):
        raise KernelError(f"latent prepare: proj {tuple(proj.shape)}, q_att {tuple(q_att.shape)}")
    if rot_dims:
        _need(inv_freq, "rotary frequencies", torch.float32)
        if inv_freq.numel() != rot_dims // 2:
            raise KernelError("latent prepare: one frequency per rotated pair is needed")
    if write_kv:
        _need(slot_mapping, "slot mapping", torch.int32)
        _need(cache, "latent cache", proj.dtype)
        _need(norm_weight, "latent norm weight", torch.float32)
        if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != rank + rot or norm_weight.numel() != rank:
            raise KernelError(f"latent prepare: cache {tuple(cache.shape)} for rows of {rank} + {rot}")
    _check(
        _lib().ferris_latent_prepare(_ptr(proj), _c_int(ld), _c_int(_dt(proj, "latent prepare")), _c_int(q_off),
                                     _c_int(dkv_off), _ptr(norm_weight), _c_float(eps), _ptr(positions), _ptr(inv_freq),
                                     _c_int(rot_dims), _ptr(slot_mapping if write_kv else None),
                                     _ptr(cache if write_kv else None), _ptr(q_att), _c_int(ldqa), _c_int(T), _c_int(heads),
                                     _c_int(dim), _c_int(rot), _c_int(rank), _c_int(1 if write_kv else 0), _stream()),
        "latent prepare",
    )


def head_gemm(x: torch.Tensor, x_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int,
              gate: Optional[torch.Tensor] = None):
    """out[t, h * out_head_stride + n] = (sum_k x[t, h * x_head_stride + k] w[h, k, n]) * g, g = sigmoid(gate[t, h]) or 1.
    ``w``: [heads, K, N] in the activations' type; fp32 sums."""
    T, wx, ldx = _rows(x, "head product input")
    T2, wo, ldo = _rows(out, "head product output")
    _need(w, "head product weights", x.dtype)
    if w.dim() != 3:
        raise KernelError(f"head product: weights {tuple(w.shape)}")
    H, K, N = w.shape
    ldg = 0
    if gate is not None:
        T3, wg, ldg = _rows(gate, "head gates")
        if T3 != T or wg != H or gate.dtype != x.dtype:
            raise KernelError(f"head product: gates {tuple(gate.shape)} for {H} heads")
    if T2 != T or out.dtype != x.dtype or (H - 1) * x_head_stride + K > wx or (H - 1) * out_head_stride + N > wo:
        raise KernelError(f"head product: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(
        _lib().ferris_head_gemm(_ptr(x), _c_int(ldx), _c_int(x_head_stride), _ptr(w), _ptr(out), _c_int(ldo),
                                _c_int(out_head_stride), _ptr(gate), _c_int(ldg), _c_int(_dt(x, "head product")), _c_int(T),
                                _c_int(H), _c_int(K), _c_int(N), _stream()),
        "head product",
    )


class RotaryTable:
    """A rotation of the first ``rotary_dim`` elements of a head by position x frequency: ``freq`` fp32 [rotary_dim / 2]
    on the device; ``interleaved``: the pairs are the elements (2i, 2i + 1), else (i, i + rotary_dim / 2);
    ``magnitude``: a factor on every cosine and sine.  ``freq_lo`` (optional, fp32 like ``freq``): what ``freq`` lacks of
    the frequencies' 64-bit values; a kernel that takes it forms position x frequency beyond 32-bit rounding."""

    __slots__ = ("freq", "rotary_dim", "interleaved", "magnitude", "freq_lo")

    def __init__(self, freq: torch.Tensor, rotary_dim: int, interleaved: bool = False, magnitude: float = 1.0,
                 freq_lo: Optional[torch.Tensor] = None):
        self.freq, self.rotary_dim = freq, int(rotary_dim)
        self.interleaved, self.magnitude = bool(interleaved), float(magnitude)
        self.freq_lo = freq_lo


def _rotary_args(rotary: Optional[RotaryTable], ctx, head_dim: int, device) -> tuple:
    """(positions, freq, rotary_dim, interleaved, magnitude) as the launchers take them; no rotation: null positions."""
    if rotary is None or rotary.rotary_dim == 0:
        return _ptr(None), _ptr(None), _c_int(0), _c_int(0), _c_float(1.0)
    _need(rotary.freq, "rotary frequencies", torch.float32)
    _need(ctx.positions, "positions", torch.int32)
    if rotary.rotary_dim % 2 or rotary.rotary_dim > head_dim or rotary.freq.numel() != rotary.rotary_dim // 2:
        raise KernelError(f"rotation of {rotary.rotary_dim} elements ({rotary.freq.numel()} frequencies) of heads of {head_dim}")
    return (_ptr(ctx.positions), _ptr(rotary.freq), _c_int(rotary.rotary_dim), _c_int(1 if rotary.interleaved else 0),
            _c_float(rotary.magnitude))


def dynamic_tanh(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor, out: torch.Tensor,
                 row_index: Optional[torch.Tensor] = None):
    """out[r] = tanh(alpha * x[row_index[r] or r]) * weight + bias, element by element in fp32 (``alpha``: one number on
    the device); x fp32, out in the activations' type."""
    _need(x, "dynamic tanh input", torch.float32)
    _need(weight, "dynamic tanh weight", torch.float32)
    _need(bias, "dynamic tanh bias", torch.float32)
    _need(alpha, "dynamic tanh alpha", torch.float32)
    _need(out, "dynamic tanh output")
    rows, H = out.shape
    if x.shape[1] != H or weight.numel() != H or bias.numel() != H or alpha.numel() != 1:
        raise KernelError(f"dynamic tanh: x {tuple(x.shape)}, weight {tuple(weight.shape)}, bias {tuple(bias.shape)}, "
                          f"alpha {tuple(alpha.shape)}")
    if row_index is not None:
        _need(row_index, "row index", torch.int32)
        if row_index.numel() != rows:
            raise KernelError("dynamic tanh: one row index per output row is needed")
    elif x.shape[0] != rows:
        raise KernelError("dynamic tanh: input and output row counts differ")
    _check(_lib().ferris_dynamic_tanh(_ptr(x), _ptr(weight), _ptr(bias), _ptr(alpha), _ptr(row_index), _ptr(out),
                                      _c_int(_dt(out, "dynamic tanh output")), _c_int(rows), _c_int(H), _stream()),
           "dynamic tanh")


def softcap_(logits: torch.Tensor, cap: float):
    """logits <- cap * tanh(logits / cap) in place; fp32."""
    _need(logits, "logits", torch.float32)
    _check(_lib().ferris_softcap(_ptr(logits), ctypes.c_longlong(logits.numel()), _c_float(cap), _stream()), "softcap")


def qk_norm_rotary_cache_write(qkv: torch.Tensor, ctx, slot_mapping: Optional[torch.Tensor], k_cache, v_cache,
                               num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                               q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                               rotary: Optional[RotaryTable], values_from_keys: bool = False, write_kv: bool = True,
                               per_head: bool = False):
    """Between the q/k(/v) product and attention: q and k each divided by the root mean square of their WHOLE projection
    (all heads at once) and multiplied by ``q_norm`` / ``k_norm`` (fp32, one number per element; None: no norm), then
    rotated by the tokens' positions; q rewritten in place, k and the values into the paged cache.
    ``values_from_keys``: the values are the keys as projected (before norm and rotation); the rows then hold
    [nh d | nkv d] only.  ``per_head``: every head is divided by the root mean square of its own elements instead, and
    the weights hold ``head_dim`` numbers that all heads share (not with ``values_from_keys``)."""
    T, width, ld = _rows(qkv, "qkv")
    want = (num_heads + num_kv_heads) * head_dim + (0 if values_from_keys else num_kv_heads * v_head_dim)
    if width != want:
        raise KernelError(f"qk norm + rotation: rows of {width} for {num_heads}+{num_kv_heads} heads of {head_dim}")
    if per_head and values_from_keys:
        raise KernelError("qk norm + rotation: the norm per head does not go with values taken from the keys")
    for name, t_, n in (("q norm weight", q_norm, head_dim if per_head else num_heads * head_dim),
                        ("k norm weight", k_norm, head_dim if per_head else num_kv_heads * head_dim)):
        if t_ is not None:
            _need(t_, name, torch.float32)
            if t_.numel() != n:
                raise KernelError(f"qk norm + rotation: {name} of {t_.numel()} for {n} elements")
    page_size = 1
    if write_kv:
        _need(slot_mapping, "slot mapping", torch.int32)
        _need(k_cache, "key cache", qkv.dtype)
        _need(v_cache, "value cache", qkv.dtype)
        page_size = k_cache.shape[2]
        if (slot_mapping.numel() != T or k_cache.shape[1:] != (num_kv_heads, page_size, head_dim)
                or v_cache.shape != (*k_cache.shape[:3], v_head_dim)):
            raise KernelError(f"qk norm + rotation: caches {tuple(k_cache.shape)} {tuple(v_cache.shape)} do not fit")
    positions, freq, rdim, inter, mag = _rotary_args(rotary, ctx, head_dim, qkv.device)
    _need(ctx.positions, "positions", torch.int32)
    if per_head:
        _check(
            _lib().ferris_qk_head_norm_rotary_cache_write(
                _ptr(qkv), _c_int(ld), _c_int(_dt(qkv, "qkv")), _ptr(ctx.positions), _ptr(slot_mapping if write_kv else None),
                _ptr(k_cache if write_kv else None), _ptr(v_cache if write_kv else None), _c_int(T), _c_int(num_heads),
                _c_int(num_kv_heads), _c_int(head_dim), _c_int(v_head_dim), _c_int(page_size), _ptr(q_norm), _ptr(k_norm),
                _c_float(eps), freq, rdim, inter, mag, _c_int(1 if write_kv else 0),
                _ptr(rotary.freq_lo if rotary is not None and rotary.rotary_dim else None), _stream()),
            "head norm + rotation + cache write",
        )
        return
    _check(
        _lib().ferris_qk_norm_rotary_cache_write(
            _ptr(qkv), _c_int(ld), _c_int(_dt(qkv, "qkv")), _ptr(ctx.positions), _ptr(slot_mapping if write_kv else None),
            _ptr(k_cache if write_kv else None), _ptr(v_cache if write_kv else None), _c_int(T), _c_int(num_heads),
            _c_int(num_kv_heads), _c_int(head_dim), _c_int(v_head_dim), _c_int(page_size), _ptr(q_norm), _ptr(k_norm),
            _c_float(eps), freq, rdim, inter, mag, _c_int(1 if values_from_keys else 0), _c_int(1 if write_kv else 0),
            _stream()),
        "qk norm + rotation + cache write",
    )


def moe_router(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], ids: torch.Tensor,
               weights: torch.Tensor, top: int, scored: Optional[dict] = None):
    """The ``top`` experts of every row of ``x`` and their weights: logits x weight^T + bias in fp32 sums, the largest
    ``top`` (lowest index among equals), softmax over those alone.  ids int32 [T, top], weights fp32 [T, top].
    ``scored`` = {"correction": fp32 [E] or None, "groups": n, "keep": n, "with_weights": n, "identity_w": fp32 [T] or
    None}: the scores are the softmax over ALL outputs, the choice is made by score + correction among the outputs of the
    ``keep`` groups (of ``groups`` equal groups of neighbours) whose best choice score is largest, and the weights are
    the chosen scores divided by their sum + 1e-20; outputs from ``with_weights`` on are identity experts, which come
    out as the index ``with_weights`` and whose weights are summed per token into ``identity_w``."""
    T, W, ldx = _rows(x, "router input")
    _need(weight, "router matrix", x.dtype)
    _need(ids, "expert ids", torch.int32)
    _need(weights, "expert weights", torch.float32)
    E = weight.shape[0]
    if weight.shape != (E, W) or ids.shape != (T, top) or weights.shape != (T, top) or (bias is not None and bias.numel() != E):
        raise KernelError(f"router: x {tuple(x.shape)}, matrix {tuple(weight.shape)}, ids {tuple(ids.shape)}")
    if bias is not None:
        _need(bias, "router bias", torch.float32)
    corr = idw = None
    groups = keep = 1
    real = E
    if scored is not None:
        corr, idw = scored.get("correction"), scored.get("identity_w")
        groups, keep, real = int(scored.get("groups", 1)), int(scored.get("keep", 1)), int(scored.get("with_weights", E))
        if corr is not None:
            _need(corr, "router correction", torch.float32)
        if idw is not None:
            _need(idw, "identity weights", torch.float32)
        if (corr is not None and corr.numel() != E) or (idw is not None and idw.numel() != T) or (real < E and idw is None):
            raise KernelError(f"router: correction / identity weights do not fit {E} outputs and {T} rows")
    _check(_lib().ferris_moe_router(_ptr(x), _c_int(ldx), _c_int(_dt(x, "router")), _ptr(weight), _ptr(bias), _ptr(ids),
                                    _ptr(weights), _c_int(T), _c_int(W), _c_int(E), _c_int(top),
                                    _c_int(0 if scored is None else 1), _ptr(corr), _c_int(groups), _c_int(keep), _c_int(real),
                                    _ptr(idw), _stream()), "router")


MOE_FEW_MAX_PAIRS = 1024  # up to here the token-major form reads an expert's weights once for all its tokens
MOE_GROUPED_MIN_TOKENS = 17  # from here on (bf16) the experts' rows are sorted by expert and meet tensor-core tiles


def moe_experts(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                h: torch.Tensor, workspace=None, accumulate: bool = True, grouped: Optional[bool] = None,
                activation: str = "silu", limit: float = 0.0, identity_w: Optional[torch.Tensor] = None):
    """h (+)= sum over a row's chosen experts of weight x down_e (silu(gate_e x) * (up_e x)).  gate_up [E, 2 ff, W] (an
    expert's gate rows, then its up rows), down [E, W, ff] in x's type; ids int32 and weights fp32 [T, top]; h fp32
    [T, W].  Steps of few tokens (up to MOE_FEW_MAX_PAIRS choices): a block per (expert, slab of rows) reads the weights
    once for all tokens that chose the expert.  More choices in 32-bit: a block per (token, chosen expert).  Both form
    whole dot products in the same order, so a token's result has the same bits.  Longer steps in bf16 (``grouped``; None = decide by size and alignment): the pairs sorted by expert, two
    tensor-core products over tiles that each meet their own expert's weights, and a pass that adds a token's results
    in the order of its choices.  ``activation``, ``limit``: the experts' gated activation (see ``gated_activation``).
    ``identity_w`` fp32 [T]: ids may then hold E, an expert that meets no weights, and h also gets identity_w[t] x[t]."""
    T, W, ldx = _rows(x, "experts input")
    if activation not in GATED_ACTIVATIONS:
        raise KernelError(f"experts: activation '{activation}' is not known ({', '.join(GATED_ACTIVATIONS)})")
    act_kind = GATED_ACTIVATIONS[activation]
    if identity_w is not None:
        _need(identity_w, "identity weights", torch.float32)
        if identity_w.numel() != T:
            raise KernelError(f"experts: {identity_w.numel()} identity weights for {T} rows")
    T2, W2, ldh = _rows(h, "experts output")
    _need(gate_up, "gate and up matrices", x.dtype)
    _need(down, "down matrices", x.dtype)
    _need(ids, "expert ids", torch.int32)
    _need(weights, "expert weights", torch.float32)
    E, ff = gate_up.shape[0], gate_up.shape[1] // 2
    top = ids.shape[1]
    if (gate_up.shape != (E, 2 * ff, W) or down.shape != (E, W, ff) or (T2, W2) != (T, W) or h.dtype != torch.float32
            or ids.shape != (T, top) or weights.shape != (T, top)):
        raise KernelError(f"experts: x {tuple(x.shape)}, gate/up {tuple(gate_up.shape)}, down {tuple(down.shape)}, "
                          f"ids {tuple(ids.shape)}")
    get = (lambda name, shape, dtype: workspace.get(name, shape, dtype)) if workspace is not None else \
        (lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=x.device))
    can_group = (x.dtype == torch.bfloat16 and W % 8 == 0 and ff % 8 == 0 and ldx % 8 == 0 and ldh % 4 == 0
                 and x.data_ptr() % 16 == 0 and h.data_ptr() % 16 == 0)
    if grouped is None:
        grouped = can_group and T >= MOE_GROUPED_MIN_TOKENS
    if grouped:
        if not can_group:
            raise KernelError("experts: the sorted form takes bf16 rows of multiples of 8 elements that start on 16 bytes")
        rows = _lib().ferris_moe_sorted_rows(_c_int(T), _c_int(top), _c_int(E + (1 if identity_w is not None else 0)))
        if rows <= 0:
            raise KernelError(f"experts: {T} tokens x {top} choices are more than one launch takes")
        pos = get("moe_pos", (T * top,), torch.int32)
        row_token = get("moe_row_token", (rows,), torch.int32)
        tile_expert = get("moe_tile_expert", (rows // 128,), torch.int32)
        xs = get("moe_sorted_rows", (rows, W), x.dtype)
        act = get("moe_sorted_act", (rows, ff), x.dtype)
        y = get("moe_sorted_out", (rows, W), torch.float32)
        _check(_lib().ferris_moe_experts_grouped(_ptr(x), _c_int(ldx), _ptr(gate_up), _ptr(down), _ptr(ids), _ptr(weights),
                                                 _ptr(h), _c_int(ldh), _c_int(T), _c_int(W), _c_int(ff), _c_int(top),
                                                 _c_int(E), _c_int(rows), _ptr(pos), _ptr(row_token), _ptr(tile_expert),
                                                 _ptr(xs), _ptr(act), _ptr(y), _c_int(1 if accumulate else 0),
                                                 _c_int(act_kind), _c_float(limit), _ptr(identity_w), _stream()),
               "experts (sorted)", 5)
        return
    act = get("moe_act", (T * top, ff), x.dtype)
    up = gate_up[:, ff:, :]
    # few pairs: the weights are read once per expert, the results of a pair stand in y until they are added
    few = 1 < T * top <= MOE_FEW_MAX_PAIRS and W % 4 == 0 and ldh % 4 == 0 and h.data_ptr() % 16 == 0
    y = get("moe_pair_out", (T * top, W), torch.float32) if few else None
    _check(_lib().ferris_moe_experts_token_major(_ptr(x), _c_int(ldx), _c_int(_dt(x, "experts")), _ptr(gate_up), _ptr(up),
                                                 ctypes.c_longlong(2 * ff * W), _ptr(down), _ptr(ids), _ptr(weights),
                                                 _ptr(act), _ptr(h), _c_int(ldh), _c_int(T), _c_int(W), _c_int(ff),
                                                 _c_int(top), _c_int(1 if accumulate else 0),
                                                 _ptr(y) if few else ctypes.c_void_p(0), _c_int(E), _c_int(act_kind),
                                                 _c_float(limit), _ptr(identity_w), _stream()),
           "experts", 3 if few else 2)


def kernel_status() -> int:
    """Reads and clears the device status word (synchronises).  0: no kernel gave up a bounded wait;
    otherwise (code << 16) | place."""
    return int(_lib().ferris_kernel_status())


def check_kernel_status() -> None:
    v = kernel_status()
    if v:
        raise KernelError(f"a kernel gave up a bounded wait (code {v >> 16}, place {v & 0xffff}); its results are wrong")


_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = max(1, _lib().ferris_sm_count())
    return _sm_count


def tensor_core_attention_takes(dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the TMA + tensor-core attention kernels take this geometry (the general kernel takes the rest)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0
            and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)


def decode_splits(tokens: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Into how many key ranges a single-token step is split, so that the GPU's SMs have work:
    one CTA per SM at most (each streams its keys through four per-warp pipelines and holds most of the
    SM's shared memory, so a CTA more than there are SMs would wait for a second round), and at least
    eight 16-key tiles per CTA."""
    base = max(1, tokens * num_kv_heads)
    want = max(1, sm_count() // base)
    most = max(1, (max_kv_len // 16) // 8)
    return max(1, min(want, most))


def decode_attention(qkv, out, k_cache, v_cache, block_tables, token_seq, positions, num_heads, num_kv_heads,
                     head_dim, window, scale, splits, scratch, rows: Optional[torch.Tensor] = None):
    """Split-KV attention for single tokens (bf16, head size 64 or 128): every row of the step, or the rows
    that ``rows`` (int32) names when the step also carries portions of prompts."""
    T, _, ldq = _rows(qkv, "attention queries")
    _, _, ldo = _rows(out, "attention output")
    n = T if rows is None else rows.numel()
    need = n * num_heads * splits * (head_dim + 2) if splits > 1 else 0
    if need and (scratch is None or scratch.numel() < need or scratch.dtype != torch.float32):
        raise KernelError(f"decode attention with {splits} splits needs {need} floats of scratch")
    common = (_ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
              ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables), _c_int(block_tables.shape[1]), _ptr(token_seq),
              _ptr(positions))
    tail = (_c_int(num_heads), _c_int(num_kv_heads), _c_int(head_dim), _c_int(k_cache.shape[2]), _c_int(window or 0),
            _c_float(scale), _c_int(splits), _ptr(scratch if need else None), _stream())
    kernels = 2 if splits > 1 else 1  # the attention kernel and the merge of its key ranges
    if rows is None:
        _check(_lib().ferris_decode_attention(*common, _c_int(T), *tail), "decode attention", kernels)
    else:
        _need(rows, "rows of the single tokens", torch.int32)
        _check(_lib().ferris_decode_attention_listed(*common, _ptr(rows), _c_int(rows.numel()), *tail), "decode attention",
               kernels)


def prefill_attention(qkv, out, k_cache, v_cache, block_tables, seq_q_start, seq_start_pos, num_seqs, max_q_len,
                      num_heads, num_kv_heads, head_dim, window, scale, skip_single: bool = False):
    """Tensor-core attention for portions of prompts (bf16, head size 64 or 128).  ``skip_single``: requests
    that bring one token are left out (the decode kernel takes them)."""
    _, _, ldq = _rows(qkv, "attention queries")
    _, _, ldo = _rows(out, "attention output")
    _check(
        _lib().ferris_prefill_attention(_ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
                                        ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables),
                                        _c_int(block_tables.shape[1]), _ptr(seq_q_start), _ptr(seq_start_pos),
                                        _c_int(num_seqs), _c_int(max_q_len), _c_int(num_heads), _c_int(num_kv_heads),
                                        _c_int(head_dim), _c_int(k_cache.shape[2]), _c_int(window or 0), _c_float(scale),
                                        _c_int(1 if skip_single else 0), _stream()),
        "prefill attention",
    )


def set_prefill_tcgen05(on=True) -> None:
    """Portions of prompts on the tcgen05 attention kernel (True / 1, the default), on the mma.sync kernel it
    replaced (False / 0), or on the tcgen05 kernel with one softmax group at every head size (2)."""
    _lib().ferris_set_prefill_tcgen05(_c_int(int(on)))


def attention_step(qkv, out, k_cache, v_cache, meta, ctx, num_heads, num_kv_heads, head_dim, inv_freq, rotary_dim,
                   window, scale, write_kv: bool = True, lazy_merge: bool = False, rotated: bool = False,
                   score_slopes: Optional[torch.Tensor] = None):
    """Everything between the q/k/v product and the output product of an attention layer: rotate q and k by
    position, put k and v into the paged cache (``meta``: the step's block tables and slots for the cache's
    page group), attend.  A step of single tokens with whole-head rotation on the tensor-core path is ONE
    kernel (the split-KV kernel rotates and writes on its way); everything else is the rotary / cache-write
    kernel followed by ``paged_attention``.  Returns ``out``; with ``lazy_merge`` it may return a
    LazySplitMerge instead (``out`` not yet written), which ``gemm`` takes as its input.  ``rotated``: the
    q/k/v product has rotated and stored already (``qkv_rope_gemm``), only attention is left.
    ``score_slopes`` (fp32 [num_heads], of a position encoding that acts on the scores): slopes[head] * (j - P) is
    added to the score of the key at position j for the query at position P; the general kernel then attends."""
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    if rotated:
        paged_attention(qkv, out, k_cache, v_cache, meta.block_tables, ctx, num_heads, num_kv_heads, head_dim, window, scale,
                        score_slopes=score_slopes)
        return out
    if (ctx.max_q_len == 1 and rotary_dim == head_dim and inv_freq is not None and score_slopes is None
            and tensor_core_attention_takes(qkv.dtype, num_heads, num_kv_heads, head_dim, page_size)):
        _need(k_cache, "key cache", qkv.dtype)
        _need(v_cache, "value cache", qkv.dtype)
        _need(meta.block_tables, "block tables", torch.int32)
        _need(meta.slot_mapping, "slot mapping", torch.int32)
        _need(inv_freq, "rotary frequencies", torch.float32)
        if (k_cache.dim() != 4 or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim
                or v_cache.shape != k_cache.shape or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim
                or out.shape != (T, num_heads * head_dim) or out.dtype != qkv.dtype
                or inv_freq.numel() != head_dim // 2 or meta.slot_mapping.numel() != T):
            raise KernelError(f"attention step: qkv {tuple(qkv.shape)}, cache {tuple(k_cache.shape)}, out {tuple(out.shape)}")
        kv_span = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        # Who merges the key ranges: with the skinny products the attention kernel itself (the ranges of a token and
        # kv head are a thread-block cluster that adds them through its shared memory); otherwise the output product
        # on its way (lazy_merge) or a merge kernel
        in_cluster = gemm_skinny_enabled()
        if in_cluster:
            splits = int(_lib().ferris_decode_cluster_splits(T, num_kv_heads, head_dim, kv_span))
            in_cluster = splits >= 1
        if not in_cluster:
            splits = decode_splits(T, num_kv_heads, kv_span)
        need = T * num_heads * splits * (head_dim + 2) if (splits > 1 and not in_cluster) else 0
        scratch = ctx.workspace.get("attn_split_scratch", (need,), torch.float32) if need else None
        leave = bool(lazy_merge and need)
        mode = 3 if in_cluster else (0 if leave else 1)
        _, _, ldq = _rows(qkv, "attention queries")
        _, _, ldo = _rows(out, "attention output")
        _check(
            _lib().ferris_decode_attention_rope(
                _ptr(qkv), _c_int(ldq), _ptr(out), _c_int(ldo), _ptr(k_cache), _ptr(v_cache),
                ctypes.c_longlong(k_cache.shape[0]), _ptr(meta.block_tables), _c_int(meta.block_tables.shape[1]),
                _ptr(ctx.token_seq), _ptr(ctx.positions), _ptr(inv_freq), _ptr(meta.slot_mapping if write_kv else None),
                _c_int(T), _c_int(num_heads), _c_int(num_kv_heads), _c_int(head_dim), _c_int(page_size),
                _c_int(window or 0), _c_float(scale), _c_int(splits), _ptr(scratch), _c_int(mode), _stream()),
            "decode attention with rotation", 2 if (splits > 1 and mode == 1) else 1,
        )
        return LazySplitMerge(scratch, out, num_heads, head_dim, splits) if leave else out
    rope_cache_write(qkv, ctx.positions, inv_freq, meta.slot_mapping, k_cache, v_cache, num_heads, num_kv_heads,
                     head_dim, rotary_dim, page_size, write_kv=write_kv)
    paged_attention(qkv, out, k_cache, v_cache, meta.block_tables, ctx, num_heads, num_kv_heads, head_dim, window, scale,
                    score_slopes=score_slopes)
    return out


def paged_attention(qkv, out, k_cache, v_cache, block_tables, ctx, num_heads, num_kv_heads, head_dim, window, scale,
                    score_slopes=None, v_head_dim: Optional[int] = None, values_in_keys: bool = False,
                    chunk: int = 0, fp32_weights: bool = False):
    """Attention of the step's tokens over the paged cache (their own keys are in it already).
    ``chunk``: see ``paged_attention_simt``.  ``fp32_weights``: the softmax's weights and the weighted sum stay in 32-bit
    (the tensor-core kernels round the weights to bf16 for their second product), so the general kernel runs.
    ``ctx`` is the step context.  bf16 with head size 64 / 128 runs on the tensor cores: the split-KV
    kernel when every request brings one token, the prefill kernel otherwise; every other geometry, the
    32-bit path, scores with slopes added (``score_slopes``) and value heads of another size than the keys'
    (``v_head_dim``) run the general kernel."""
    _need(k_cache, "key cache", qkv.dtype)
    if isinstance(score_slopes, ScoreTerms) and not score_slopes.any():
        score_slopes = None
    if values_in_keys or chunk or fp32_weights or (v_head_dim is not None and v_head_dim != head_dim):
        paged_attention_simt(qkv, out, k_cache, v_cache, block_tables, ctx.token_seq, ctx.positions, num_heads,
                             num_kv_heads, head_dim, window, scale, score_slopes=score_slopes, v_head_dim=v_head_dim,
                             max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, workspace=ctx.workspace,
                             values_in_keys=values_in_keys, chunk=chunk)
        return
    _need(v_cache, "value cache", qkv.dtype)
    _need(block_tables, "block tables", torch.int32)
    if k_cache.dim() != 4 or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim \
            or v_cache.shape != k_cache.shape or block_tables.dim() != 2:
        raise KernelError(f"attention: cache {tuple(k_cache.shape)}, tables {tuple(block_tables.shape)}")
    if out.dtype != qkv.dtype or out.shape[1] != num_heads * head_dim or out.shape[0] != qkv.shape[0]:
        raise KernelError(f"attention: q {tuple(qkv.shape)}, out {tuple(out.shape)}")
    if score_slopes is not None or not tensor_core_attention_takes(qkv.dtype, num_heads, num_kv_heads, head_dim, k_cache.shape[2]):
        paged_attention_simt(qkv, out, k_cache, v_cache, block_tables, ctx.token_seq, ctx.positions, num_heads,
                             num_kv_heads, head_dim, window, scale, score_slopes=score_slopes, max_q_len=ctx.max_q_len,
                             max_kv_len=ctx.max_kv_len, workspace=ctx.workspace)
        return
    T = qkv.shape[0]
    singles = getattr(ctx, "single_rows", None)
    if ctx.max_q_len == 1 or singles is not None:
        # single tokens: all rows of the step, or the listed ones beside portions of prompts
        n = T if ctx.max_q_len == 1 else singles.numel()
        kv_span = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        splits = decode_splits(n, num_kv_heads, kv_span)
        scratch = None
        if splits > 1:
            scratch = ctx.workspace.get("attn_split_scratch", (n * num_heads * splits * (head_dim + 2),), torch.float32)
        decode_attention(qkv, out, k_cache, v_cache, block_tables, ctx.token_seq, ctx.positions, num_heads,
                         num_kv_heads, head_dim, window, scale, splits, scratch,
                         rows=None if ctx.max_q_len == 1 else singles)
    if ctx.max_q_len > 1:
        prefill_attention(qkv, out, k_cache, v_cache, block_tables, ctx.seq_q_start, ctx.seq_start_pos, ctx.num_seqs,
                          ctx.max_q_len, num_heads, num_kv_heads, head_dim, window, scale,
                          skip_single=singles is not None)


def sample(logits: torch.Tensor, out_token: torch.Tensor, out_prob: Optional[torch.Tensor] = None,
           temperature: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
           rng_states: Optional[torch.Tensor] = None):
    """One token per row of fp32 ``logits`` [n, V].  Without ``temperature``: argmax (lowest index on
    ties).  With it: per-row temperature, top_k (<= 0: whole vocabulary), top_p, and one draw from
    ``rng_states[slots[row]]`` (int64 xorshift64* states, advanced in place)."""
    n, V, ld = _rows(logits, "logits")
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _need(out_token, "sampled tokens", torch.int32)
    if out_token.numel() != n:
        raise KernelError("sample: one output token per row is needed")
    if out_prob is not None:
        _need(out_prob, "sample probabilities", torch.float32)
    if temperature is not None:
        _need(temperature, "temperatures", torch.float32)
        _need(top_k, "top_k", torch.int32)
        _need(top_p, "top_p", torch.float32)
        _need(slots, "generator slots", torch.int32)
        _need(rng_states, "generator states", torch.int64)
        if not (temperature.numel() == top_k.numel() == top_p.numel() == slots.numel() == n):
            raise KernelError("sample: one temperature, top_k, top_p and slot per row is needed")
    _check(
        _lib().ferris_sample(_ptr(logits), _c_int(ld), _c_int(n), _c_int(V), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                             _ptr(slots), _ptr(rng_states), _ptr(out_token), _ptr(out_prob), _stream()),
        "sample",
    )

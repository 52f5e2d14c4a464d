"""Python face of the sm_100a kernels.

Each function checks its tensors, then calls one ``extern "C"`` launcher of the
compiled library on the current CUDA stream.  There is no other implementation
behind these names: a tensor that is not on a CUDA device, or a library that
cannot be built, raises.

bfloat16 matrix products run hand-written kernels: a weight-streaming product
for the few rows of a decode step and tcgen05 products (one SM or a pair of SMs
per tile) for prompt portions; only the row counts between them call the library
GEMM (cuBLAS through ``torch.mm``), which the reference's engine calls for every
linear layer (``F.linear``, ``ops/attention.py:128-130``, ``ops/mlp.py:117,128``,
``ops/embedding.py:92``).  float32 products run the hand-written FMA kernel, never
a tensor-core mode.
"""

from __future__ import annotations

import ctypes
import functools

import torch

from .build import KernelBuildError, load_library

_CORE_SOURCES = ["rowwise.cu", "rope_kv.cu", "gemm_fp32.cu", "gemm_skinny.cu", "gemm_tc.cu", "gemm_tc2.cu",
                 "attention_generic.cu", "sampling.cu"]

_ERRORS = {
    -1: "bad argument (null pointer, negative size or misaligned pointer)",
    -2: "a size this kernel does not take",
    -3: "a dtype this kernel does not take",
    -4: "a size beyond the kernel's stated maximum",
}

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def core_sources() -> list[str]:
    from .build import CSRC
    return [s for s in _CORE_SOURCES if (CSRC / s).is_file()]


_core_lib: ctypes.CDLL | None = None
_attention_libs: dict[int, ctypes.CDLL] = {}


def core() -> ctypes.CDLL:
    """The library of all kernels that do not depend on the head size (built at first use)."""
    global _core_lib
    if _core_lib is None:
        _core_lib = load_library("si_core", core_sources())
    return _core_lib


ATTENTION_SOURCES = ["attention_mma.cu", "attention_tc.cu"]


def attention_library(head_dim: int) -> ctypes.CDLL:
    """Tensor-core attention kernels are compiled for one head size at a time."""
    lib = _attention_libs.get(head_dim)
    if lib is None:
        if head_dim % 16 != 0 or not (16 <= head_dim <= 256):
            raise KernelError(
                f"head_dim {head_dim}: the attention kernels take multiples of 16 from 16 to 256"
            )
        lib = load_library(f"si_attn_d{head_dim}", ATTENTION_SOURCES,
                           [f"-DSI_HEAD_DIM={head_dim}"])
        _attention_libs[head_dim] = lib
    return lib


launch_count = 0  # kernels of this package launched so far (a graph replay is counted by its owner)


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: refused, {_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not float32 or bfloat16")


def _dev(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("kernel called with a tensor that is not on a CUDA device; "
                              "there is no CPU path")
        if not t.is_contiguous():
            raise KernelError(f"kernel called with a non-contiguous tensor of shape {tuple(t.shape)}")


def _p(t: torch.Tensor | None) -> ctypes.c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


# The current stream's handle, asked for once per kernel launch: torch's own binding for it costs
# a fraction of a microsecond, torch.cuda.current_stream() (device look-ups, an object per call)
# some ten times that, which showed as a third of the host time of a step of 250 launches.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    if _raw_stream is not None and _raw_device is not None:
        return _c_void_p(_raw_stream(_raw_device()))
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _i32(t: torch.Tensor | None, name: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, is {t.dtype}")


# ----------------------------------------------------------------- row-wise

def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` as float32 (the residual stream)."""
    _dev(table, ids, out)
    _i32(ids, "ids")
    n, hidden = out.shape
    if out.dtype != torch.float32 or table.shape[1] != hidden or ids.numel() < n:
        raise KernelError("embed_gather: shape or dtype mismatch")
    _check(core().si_embed_gather(_p(table), _dt(table), _p(ids), _p(out), n, hidden,
                                  table.shape[0], _stream()), "embed_gather")
    return out


class PartialSums:
    """The output of a product whose k-range was cut across blocks: float32 slices
    ``[splits, rows, width]`` that whoever consumes them adds up, in order, and rounds to
    ``dtype`` (what the product would have stored had it not been cut).  ``rmsnorm`` takes one
    in place of ``delta``; ``tensor()`` is the sum for everyone else."""

    def __init__(self, slices: torch.Tensor, dtype: torch.dtype):
        self.slices = slices
        self.dtype = dtype
        self.shape = tuple(slices.shape[1:])

    def tensor(self) -> torch.Tensor:
        total = self.slices[0].clone()
        for p in range(1, self.slices.shape[0]):
            total += self.slices[p]
        return total.to(self.dtype)


def rmsnorm(residual: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: "torch.Tensor | PartialSums | None" = None,
            rows: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of rows of the float32 residual, with the pending add fused in.

    Without ``rows``: ``residual += delta`` (if given) in place, ``out = norm(residual)``.
    With ``rows``: ``out[r] = norm(residual[rows[r]] + delta[rows[r]])``, residual untouched.
    ``delta`` may be the ``PartialSums`` of a product.
    """
    parts = None
    if isinstance(delta, PartialSums):
        parts, delta = delta.slices, None
    _dev(residual, weight, out, delta, rows, parts)
    _i32(rows, "rows")
    n_rows, hidden = out.shape
    if residual.dtype != torch.float32 or residual.shape[1] != hidden or weight.numel() != hidden:
        raise KernelError("rmsnorm: shape or dtype mismatch")
    if delta is not None and (delta.dtype != out.dtype or delta.shape[1] != hidden):
        raise KernelError("rmsnorm: delta must have the dtype of out and the width of residual")
    if parts is not None and (parts.dtype != torch.float32 or parts.dim() != 3 or
                              parts.shape[2] != hidden):
        raise KernelError("rmsnorm: partial sums must be float32 [splits, rows, width of residual]")
    if rows is None and residual.shape[0] < n_rows:
        raise KernelError("rmsnorm: fewer residual rows than output rows")
    if rows is not None and rows.numel() < n_rows:
        raise KernelError("rmsnorm: fewer row indices than output rows")
    _check(core().si_rmsnorm(_p(residual), _p(delta), _p(parts),
                             0 if parts is None else parts.shape[0],
                             ctypes.c_longlong(0 if parts is None else parts.stride(0)),
                             _p(weight), _p(rows), _p(out), n_rows,
                             hidden, _c_float(eps), _dt(out), _dt(weight), _stream()), "rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]`` in float32 arithmetic."""
    _dev(gate_up, out)
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: shape or dtype mismatch")
    _check(core().si_swiglu(_p(gate_up), _p(out), n, inter, _dt(out), _stream()), "swiglu")
    return out


# ------------------------------------------------------------ matrix product

SKINNY_MAX_ROWS = 16  # up to this many tokens the hand-written weight-streaming product runs
TENSOR_CORE_MIN_ROWS = 96  # from this many tokens the tcgen05 product runs (its tiles have 128 rows)

_status: dict[int, torch.Tensor] = {}  # per device: one int the tcgen05 kernels write on a time-out
_STATUS_TEXT = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue"}


def status_tensor(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: torch.device | None = None) -> None:
    """Raise if a tcgen05 kernel gave up waiting on a barrier (synchronises the device)."""
    for idx, t in list(_status.items()):
        if device is not None and device.index not in (None, idx):
            continue
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise KernelError(f"tcgen05 matrix product on cuda:{idx}: {_STATUS_TEXT.get(code, code)} "
                              f"waited over a second for a barrier and gave up; results are invalid")


def _tc_ok(x: torch.Tensor, weight: torch.Tensor, n_out: int) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] >= TENSOR_CORE_MIN_ROWS
            and x.shape[1] % 8 == 0 and n_out % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


PAIRED_MIN_ROWS = 256  # from this many rows a tile of 256 rows on a pair of SMs is full


def linear_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, swiglu: bool = False,
              paired: bool | None = None) -> torch.Tensor:
    """The tcgen05 product: ``out = x @ weight.T`` (bfloat16), or its SwiGLU form.

    ``paired``: run on pairs of SMs (256-row tiles); by default from 256 rows on."""
    _dev(x, weight, out)
    m, k = x.shape
    n = out.shape[1]
    if out.dtype != torch.bfloat16 or out.shape[0] != m or weight.shape != ((2 * n if swiglu else n), k) \
            or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0:
        raise KernelError("linear_tc: operands do not fit")
    if paired is None:
        paired = m >= PAIRED_MIN_ROWS
    fn = core().si_gemm_tc2_bf16 if paired else core().si_gemm_tc_bf16
    _check(fn(_p(x), x.stride(0), _p(weight), _p(out), out.stride(0), m, n, k,
              2 if swiglu else 0, _p(status_tensor(x.device)), _stream()),
           "gemm_tc2" if paired else "gemm_tc")
    return out


def _skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and 0 < x.shape[0] <= SKINNY_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = x @ weight.T`` for ``weight`` in the ``[out, in]`` layout.

    float32 operands: the FMA kernel (true 32-bit).  bfloat16 operands: up to 16
    rows the weight-streaming kernel, from 96 rows the tcgen05 kernel, between
    them (and for float32 output above 16 rows) the library GEMM; float32
    accumulation in every case; ``out`` may be bfloat16 or float32.
    """
    _dev(x, weight, out)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or out.shape != (m, n) or x.dtype != weight.dtype:
        raise KernelError(f"linear: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> "
                          f"{tuple(out.shape)} or dtypes do not fit")
    if x.dtype == torch.float32:
        if out.dtype != torch.float32:
            raise KernelError("linear: float32 operands need a float32 output")
        _check(core().si_gemm_fp32_tn(_p(x), _p(weight), _p(out), m, n, k, k, k, n, _stream()),
               "gemm_fp32")
    elif _skinny_ok(x, weight):
        _check(core().si_gemm_skinny_bf16(_p(x), x.stride(0), _p(weight), _p(out), out.stride(0),
                                          m, n, k, 0 if out.dtype == torch.bfloat16 else 1,
                                          _stream()), "gemm_skinny")
    elif out.dtype == torch.bfloat16 and _tc_ok(x, weight, n) and out.stride(0) % 8 == 0:
        linear_tc(x, weight, out)
    elif out.dtype == torch.bfloat16:
        torch.mm(x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    return out


def linear_for_residual(x: torch.Tensor, weight: torch.Tensor, ws, tag: str,
                        partial_ok: bool) -> "torch.Tensor | PartialSums":
    """``x @ weight.T`` for a product whose output is only ever added to the residual stream.

    With few rows and a consumer that takes them (``partial_ok``), the weight-streaming kernel
    cuts the k-range across blocks so that a narrow matrix still keeps every SM fetching, and
    returns ``PartialSums``; so does the tcgen05 kernel on pairs of SMs where a product of a few
    hundred rows has too few tiles for the pairs; otherwise an ordinary tensor in ``x``'s dtype.  ``ws`` is the
    step's workspace, ``tag`` names the buffers.
    """
    m, k = x.shape
    n = weight.shape[0]
    if partial_ok and _skinny_ok(x, weight):
        splits = core().si_gemm_skinny_splits(n, k)
        if splits > 1:
            _dev(x, weight)
            if weight.shape[1] != k or x.dtype != weight.dtype:
                raise KernelError("linear_for_residual: shapes or dtypes do not fit")
            slices = ws.get(tag + ".parts", (SKINNY_MAX_SPLITS * SKINNY_MAX_ROWS, n), torch.float32,
                            row_cap=SKINNY_MAX_SPLITS * SKINNY_MAX_ROWS)
            slices = slices[:splits * m].view(splits, m, n)
            _check(core().si_gemm_skinny_bf16(_p(x), x.stride(0), _p(weight), _p(slices), n,
                                              m, n, k, 4, _stream()), "gemm_skinny_partial")
            return PartialSums(slices, x.dtype)
    if partial_ok and _tc_ok(x, weight, n):   # from 96 rows on
        # few 256-row tiles for the pairs of SMs: cut K across them where that pays
        splits = min(core().si_gemm_tc2_splits(m, n, k), max(WIDE_PART_ROWS // m, 1))
        if splits > 1:
            _dev(x, weight)
            if weight.shape[1] != k or x.dtype != weight.dtype:
                raise KernelError("linear_for_residual: shapes or dtypes do not fit")
            slices = ws.get(tag + ".wide_parts", (splits * m, n), torch.float32,
                            row_cap=WIDE_PART_ROWS).view(splits, m, n)
            _check(core().si_gemm_tc2_partial(_p(x), x.stride(0), _p(weight), _p(slices), n, m, n, k,
                                              splits, _p(status_tensor(x.device)), _stream()),
                   "gemm_tc2_partial")
            return PartialSums(slices, x.dtype)
    out = ws.get(tag, (m, n), x.dtype)
    return linear(x, weight, out)


WIDE_PART_ROWS = 4096   # rows of float32 slices kept for a tcgen05 product cut along k (all slices together)
SKINNY_MAX_SPLITS = 8   # most k-ranges the weight-streaming product cuts a matrix into


def can_fuse_swiglu(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``linear_swiglu`` can run for these operands: bfloat16 on the GPU, and either
    few rows (weight-streaming kernel) or many (tcgen05 kernel)."""
    return _skinny_ok(x, weight) or _tc_ok(x, weight, weight.shape[0] // 2)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = silu(x @ Wg.T) * (x @ Wu.T)`` with ``w_gate_up = [Wg; Wu]``, in one kernel."""
    _dev(x, w_gate_up, out)
    m, k = x.shape
    inter = out.shape[1]
    if w_gate_up.shape != (2 * inter, k) or out.shape[0] != m or out.dtype != torch.bfloat16 \
            or not can_fuse_swiglu(x, w_gate_up):
        raise KernelError("linear_swiglu: operands do not fit (see can_fuse_swiglu)")
    if not _skinny_ok(x, w_gate_up):
        return linear_tc(x, w_gate_up, out, swiglu=True)
    _check(core().si_gemm_skinny_bf16(_p(x), x.stride(0), _p(w_gate_up), _p(out), out.stride(0),
                                      m, inter, k, 2, _stream()), "gemm_skinny_swiglu")
    return out


# ------------------------------------------------------ positions and cache

def rope_kv_store(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                  kv_slots: torch.Tensor | None, pool: torch.Tensor | None, num_q_heads: int,
                  num_kv_heads: int, head_dim: int, page_size: int, write_kv: bool) -> None:
    """Rotate q (in place) and k, and write k, v of every token into its page slot."""
    _dev(qkv, positions, inv_freq, kv_slots, pool)
    _i32(positions, "positions")
    _i32(kv_slots, "kv_slots")
    n = qkv.shape[0]
    if qkv.shape[1] != (num_q_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("rope_kv_store: qkv width does not fit the head counts")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2:
        raise KernelError("rope_kv_store: inv_freq must be float32 of head_dim/2 entries")
    if write_kv:
        if pool is None or kv_slots is None or pool.dtype != qkv.dtype:
            raise KernelError("rope_kv_store: pool and kv_slots needed, pool in qkv's dtype")
        if tuple(pool.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
            raise KernelError(f"rope_kv_store: pool shape {tuple(pool.shape)} does not fit")
    _check(core().si_rope_kv_store(_p(qkv), _p(positions), _p(inv_freq), _p(kv_slots), _p(pool), n,
                                   num_q_heads, num_kv_heads, head_dim, page_size,
                                   1 if write_kv else 0, _dt(qkv), _stream()), "rope_kv_store")


def can_fuse_projection_rope(x: torch.Tensor, weight: torch.Tensor, qkv: torch.Tensor) -> bool:
    """Whether ``linear_rope_kv_store`` takes these operands: bfloat16 and few enough rows for
    the weight-streaming kernel."""
    return _skinny_ok(x, weight) and qkv.dtype == torch.bfloat16


def linear_rope_kv_store(x: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor,
                         positions: torch.Tensor, inv_freq: torch.Tensor,
                         kv_slots: torch.Tensor | None, pool: torch.Tensor | None,
                         num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         write_kv: bool) -> None:
    """``linear(x, w_qkv)`` and ``rope_kv_store`` in one kernel, for up to 16 tokens.

    Rotated queries land in the first ``num_q_heads*head_dim`` columns of ``qkv``; keys and
    values go to the pool only (the other columns of ``qkv`` are not written)."""
    _dev(x, w_qkv, qkv, positions, inv_freq, kv_slots, pool)
    _i32(positions, "positions")
    _i32(kv_slots, "kv_slots")
    m, k = x.shape
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    if not can_fuse_projection_rope(x, w_qkv, qkv) or w_qkv.shape != (width, k) \
            or qkv.shape != (m, width) or w_qkv.dtype != torch.bfloat16 or positions.numel() < m:
        raise KernelError("linear_rope_kv_store: operands do not fit (see can_fuse_projection_rope)")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2:
        raise KernelError("linear_rope_kv_store: inv_freq must be float32 of head_dim/2 entries")
    if write_kv:
        if pool is None or kv_slots is None or pool.dtype != qkv.dtype or kv_slots.numel() < m:
            raise KernelError("linear_rope_kv_store: pool and kv_slots needed, pool in qkv's dtype")
        if tuple(pool.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
            raise KernelError(f"linear_rope_kv_store: pool shape {tuple(pool.shape)} does not fit")
    _check(core().si_gemm_skinny_rope_kv_bf16(
        _p(x), x.stride(0), _p(w_qkv), _p(qkv), qkv.stride(0), m, k, _p(positions), _p(inv_freq),
        _p(kv_slots), _p(pool), num_q_heads, num_kv_heads, head_dim, page_size,
        1 if write_kv else 0, _stream()), "gemm_skinny_rope_kv")


# ---------------------------------------------------------------- attention

def attention_generic(q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                      tok_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                      num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                      window: int | None) -> torch.Tensor:
    """Attention of every token over its request's pages, float32 arithmetic.

    ``q`` may be the fused qkv buffer: only its first ``num_q_heads*head_dim``
    columns are read, with its own row stride.
    """
    _dev(pool, block_table, tok_seq, positions, out)
    if not q.is_cuda or q.stride(1) != 1:
        raise KernelError("attention: q must be a CUDA tensor with unit inner stride")
    _i32(block_table, "block_table"); _i32(tok_seq, "tok_seq"); _i32(positions, "positions")
    n = out.shape[0]
    page_size = pool.shape[3]
    if tuple(pool.shape[1:]) != (2, num_kv_heads, page_size, head_dim) or pool.dtype != q.dtype \
            or out.dtype != q.dtype:
        raise KernelError("attention: pool/out shape or dtype does not fit")
    _check(core().si_attention_generic(
        _p(q), q.stride(0), _p(pool), _p(block_table), block_table.stride(0), _p(tok_seq),
        _p(positions), _p(out), out.stride(0), n, num_q_heads, num_kv_heads, head_dim, page_size,
        _c_float(scale), int(window or 0), _dt(q), _stream()), "attention_generic")
    return out


MAX_KV_SPLITS = 32
# Cost model of the decode-attention kernel: a block costs a fixed part plus a part per
# 64-key tile, the blocks run in waves of as many as fit on the GPU (3 per SM), and joining the
# splits costs a little more with each split.  The constants are timings of heads of 128 (1 to
# 64 sequences, 512 to 8192 keys, 1 to 8 kv heads); a tile's part is its bytes and scales
# with the head size.
_RESIDENT_BLOCKS = 3 * 148
_BLOCK_US, _TILE_US_AT_128, _MERGE_US, _MERGE_SPLIT_US = 6.0, 0.8, 2.0, 0.3


@functools.lru_cache(maxsize=4096)
def _plan_kv_splits(base: int, tiles: int, head_dim: int) -> int:
    tile_us = _TILE_US_AT_128 * head_dim / 128.0
    best, best_t = 1, float("inf")
    for s in range(1, min(MAX_KV_SPLITS, tiles) + 1):
        per = -(-tiles // s)
        waves = -(-base * s // _RESIDENT_BLOCKS)
        t = waves * (_BLOCK_US + per * tile_us)
        if s > 1:
            t += _MERGE_US + s * _MERGE_SPLIT_US
        if t < best_t - 1e-9:
            best, best_t = s, t
    return best


def plan_kv_splits(n_single: int, num_q_heads: int, num_kv_heads: int, max_kv_len: int,
                   head_dim: int = 128) -> int:
    """How many blocks share the keys of one (sequence, kv head) in the decode kernel:
    the number that the cost model above makes cheapest."""
    group = num_q_heads // num_kv_heads
    base = max(1, n_single * num_kv_heads * ((group + 15) // 16))
    tiles = max(1, (max_kv_len + 63) // 64)
    return _plan_kv_splits(base, tiles, head_dim)


def paged_attention(q: torch.Tensor, pool: torch.Tensor, ctx, plan, group: int, out: torch.Tensor,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                    window: int | None) -> torch.Tensor:
    """Attention of a step's tokens over the pages of layer group ``group``.

    ``ctx`` is the step's ``StepContext``, ``plan`` its ``AttentionStepPlan``
    (``parts/attention_plan.py``; not needed in float32).  float32: the generic kernel
    for every token.  bfloat16: tensor-core kernels, one for sequences that bring a
    single token (keys split over blocks, partial results joined through scratch
    memory) and one for longer portions (64-query or 128-query tiles).
    """
    table = ctx.block_tables[group]
    if q.dtype == torch.float32:
        return attention_generic(q, pool, table, ctx.tok_seq, ctx.positions, out, num_q_heads,
                                 num_kv_heads, head_dim, scale, window)
    _dev(pool, table, out)
    if not q.is_cuda or q.stride(1) != 1 or q.dtype != torch.bfloat16:
        raise KernelError("attention: q must be a bfloat16 CUDA tensor with unit inner stride")
    page_size = pool.shape[3]
    if tuple(pool.shape[1:]) != (2, num_kv_heads, page_size, head_dim) or \
            pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention: pool/out shape or dtype does not fit")
    lib = attention_library(head_dim)
    win = int(window or 0)
    if plan.n_tiles and wide_prefill_fits(plan, head_dim, page_size):
        attention_prefill_wide(q, pool, ctx, plan, group, out, num_q_heads, num_kv_heads, head_dim,
                               scale, window)
    elif plan.n_tiles:
        _check(lib.si_attn_prefill(
            _p(q), q.stride(0), _p(pool), _p(table), table.stride(0), _p(ctx.cu_q),
            _p(ctx.positions), _p(plan.tile_seq), _p(plan.tile_start), _p(plan.tile_pairs),
            plan.n_pairs, _p(out),
            out.stride(0), num_q_heads, num_kv_heads, page_size, _c_float(scale), win, _stream()),
            "attn_prefill")
    if plan.n_single:
        n_splits = plan_kv_splits(plan.n_single, num_q_heads, num_kv_heads, ctx.max_kv_len, head_dim)
        scratch = None
        if n_splits > 1:
            scratch = ctx.ws.get("attn.split",
                                 (plan.n_single, num_q_heads * MAX_KV_SPLITS * (head_dim + 2)),
                                 torch.float32, row_cap=ctx.max_seqs)
        _check(lib.si_attn_decode(
            _p(q), q.stride(0), _p(pool), pool.shape[0], _p(table), table.stride(0), _p(ctx.cu_q),
            _p(ctx.positions), _p(plan.single_seqs), plan.n_single, _p(out), out.stride(0),
            _p(scratch), num_q_heads, num_kv_heads, page_size, _c_float(scale), win, n_splits,
            _stream()), "attn_decode", kernels=2 if n_splits > 1 else 1)
    return out


WIDE_MIN_QUERIES = 64  # shorter portions stay on the 64-query mma.sync tiles


def wide_prefill_fits(plan, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this step's portions: it is written for heads
    of 128 and 64 and pages of 8, 16, 32 or 64 tokens, and pays off from 64 queries a portion."""
    return head_dim in (64, 128) and page_size in (8, 16, 32, 64) and \
        plan.n_wide > 0 and plan.max_q_len >= WIDE_MIN_QUERIES


def attention_prefill_wide(q: torch.Tensor, pool: torch.Tensor, ctx, plan, group: int,
                           out: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                           scale: float, window: int | None) -> torch.Tensor:
    """The tcgen05 prefill kernel on the step's 128-query tiles (``plan.wide_seq/wide_start``).

    ``q`` is the query part of the fused projection output, a view with its row stride.
    """
    table = ctx.block_tables[group]
    _dev(pool, table, out)
    page_size = pool.shape[3]
    if not q.is_cuda or q.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or \
            q.stride(1) != 1 or tuple(pool.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
        raise KernelError("attention_prefill_wide: bfloat16 q, pool and out of fitting shapes")
    lib = attention_library(head_dim)
    if not lib.si_attn_prefill_tc_supported():
        raise KernelError(f"attention_prefill_wide: no tcgen05 kernel for head size {head_dim}")
    _check(lib.si_attn_prefill_tc(
        _p(q), q.stride(0), q.shape[0], _p(pool), pool.shape[0], _p(table), table.stride(0),
        _p(ctx.cu_q), _p(ctx.positions), _p(plan.wide_seq), _p(plan.wide_start), plan.n_wide, _p(out),
        out.stride(0), num_q_heads, num_kv_heads, page_size, _c_float(scale), int(window or 0),
        _stream()), "attn_prefill_tc")
    return out


# ----------------------------------------------------------------- sampling

def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seed: torch.Tensor, stream_id: torch.Tensor,
           counter: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One token per row of float32 logits; per-row parameters (see sampling.cu).  The rows of
    ``logits`` may be further apart than the vocabulary is wide."""
    _dev(temperature, top_k, top_p, seed, stream_id, counter, out)
    if not logits.is_cuda or logits.dim() != 2 or logits.stride(1) != 1 or logits.device != out.device:
        raise KernelError("sample: logits must be a matrix on the GPU of its parameters, rows contiguous")
    n, vocab = logits.shape
    if logits.dtype != torch.float32 or temperature.dtype != torch.float32 or \
            top_p.dtype != torch.float32:
        raise KernelError("sample: logits, temperature and top_p must be float32")
    for name, t in (("top_k", top_k), ("seed", seed), ("stream_id", stream_id),
                    ("counter", counter), ("out", out)):
        _i32(t, name)
        if t.numel() < n:
            raise KernelError(f"sample: {name} has fewer than {n} entries")
    _check(core().si_sample(_p(logits), n, vocab, logits.stride(0), _p(temperature), _p(top_k),
                            _p(top_p), _p(seed), _p(stream_id), _p(counter), _p(out), _stream()),
           "sample")
    return out


__all__ = ["KernelError", "KernelBuildError", "embed_gather", "rmsnorm", "swiglu", "linear", "linear_swiglu", "linear_tc",
           "linear_for_residual", "PartialSums",
           "can_fuse_swiglu", "check_status", "status_tensor",
           "rope_kv_store", "can_fuse_projection_rope", "linear_rope_kv_store", "attention_generic", "paged_attention", "attention_prefill_wide", "wide_prefill_fits", "plan_kv_splits", "sample", "core", "attention_library"]

"""Python side of the CUDA kernels: one function per launcher in ``csrc/``.

Every function takes CUDA tensors, launches on torch's current stream and raises on
any error.  There is no CPU path and no library fallback here: a tensor that is not
on a CUDA device, or a kernel library that cannot be built or loaded, is an error.
"""
from __future__ import annotations

import ctypes
import os as _os
from typing import Optional

import torch

from .csrc.build import library, loaded as _library_loaded

F32, BF16 = 0, 1
ERR_UNSUPPORTED = 10001


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device (there is no CPU path)")
    return ctypes.c_void_p(t.data_ptr())


_launch_count = [0]


def launches() -> int:
    """How many kernels of this package have been launched (replays of captured steps included)."""
    return _launch_count[0]


def add_launches(n: int) -> None:
    _launch_count[0] += n


_step_stream = [None]


class step_stream:
    """Within this context every launcher uses the stream that was current on entry, looked up once:
    asking torch for the current stream costs several microseconds, a step has hundreds of launches.
    (Nothing inside a step switches streams; a graph capture enters the context after it has begun.)"""

    def __enter__(self):
        self.previous = _step_stream[0]
        _step_stream[0] = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        _step_stream[0] = self.previous
        return False


def _stream():
    _launch_count[0] += 1          # every launcher fetches the stream exactly once
    s = _step_stream[0]
    return s if s is not None else ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code == ERR_UNSUPPORTED:
        raise KernelError(f"{what}: the kernel refuses these sizes or types")
    raise KernelError(f"{what}: CUDA error {code}")


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_I, _LL, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


# ------------------------------------------------------------------ elementwise
def embedding(x_out: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor) -> None:
    """x_out[t, :] = table[tokens[t], :]; x_out float32 [T, D], tokens int32 [T]."""
    T, D = x_out.shape
    assert x_out.dtype == torch.float32 and tokens.dtype == torch.int32 and table.shape[1] == D
    _contig(x_out, "x_out"); _contig(table, "table")
    _check(library("elementwise").qd_embedding(_ptr(x_out), _ptr(table), _I(dtype_code(table.dtype)),
                                               _ptr(tokens), _I(T), _I(D), _stream()), "embedding")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
    """out[r] = rmsnorm(x[s] + delta[s]) * weight with s = rows[r] (or r); x float32 [T, D] is
    updated to x + delta when ``write_back``."""
    D = x.shape[1]
    n_rows = out.shape[0]
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == D
    assert out.shape[1] == D and (rows is None or (rows.dtype == torch.int32 and rows.numel() == n_rows))
    assert rows is not None or n_rows == x.shape[0]
    _contig(x, "x"); _contig(out, "out")
    n_parts = 1
    if delta is not None:
        # delta [T, D], or float32 partial sums [n_parts, T, D] that the kernel adds up
        if delta.dim() == 3:
            n_parts = delta.shape[0]
            assert delta.dtype == torch.float32 and tuple(delta.shape[1:]) == tuple(x.shape)
        else:
            assert delta.shape == x.shape
        _contig(delta, "delta")
    _check(library("elementwise").qd_add_rmsnorm(
        _ptr(x), _ptr(delta), _I(dtype_code(delta.dtype) if delta is not None else -1), _ptr(weight),
        _ptr(out), _I(dtype_code(out.dtype)), _ptr(rows), _I(n_rows), _I(D), _F(eps),
        _I(1 if write_back else 0), _I(n_parts), _LL(x.numel()), _stream()), "add_rmsnorm")


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    """x += delta (delta [T, D], or float32 partial sums [n_parts, T, D])."""
    n_parts = delta.shape[0] if delta.dim() == 3 else 1
    assert x.dtype == torch.float32 and tuple(x.shape) == tuple(delta.shape[-2:])
    _contig(x, "x"); _contig(delta, "delta")
    _check(library("elementwise").qd_residual_add(_ptr(x), _ptr(delta), _I(dtype_code(delta.dtype)),
                                                  _LL(x.numel()), _I(n_parts), _stream()), "residual_add")


def rope_kv_write_partial(part: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor, H: int, G: int,
                          d: int, rotary_dim: int, pairing: int, cos: Optional[torch.Tensor],
                          sin: Optional[torch.Tensor], positions: torch.Tensor, kv: Optional[torch.Tensor],
                          slot_map: Optional[torch.Tensor], page_size: int, write_kv: bool) -> None:
    """As ``rope_kv_write`` from float32 partial sums part [n_parts, T, (H+2G)*d] (+ bias): rotated q goes
    to q_out bfloat16 [T, H*d], k and v to the cache."""
    n_parts, T, W = part.shape
    assert part.dtype == torch.float32 and W == (H + 2 * G) * d and q_out.shape == (T, H * d)
    assert q_out.dtype == torch.bfloat16 and positions.dtype == torch.int32
    _contig(part, "part"); _contig(q_out, "q_out")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == W
    if write_kv:
        assert kv.dtype == torch.bfloat16 and tuple(kv.shape[1:]) == (2, G, page_size, d)
        _contig(kv, "kv")
    _check(library("elementwise").qd_rope_kv_write_partial(
        _ptr(part), _I(n_parts), _ptr(bias), _ptr(q_out), _I(T), _I(H), _I(G), _I(d), _I(rotary_dim),
        _I(pairing), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(kv), _ptr(slot_map), _I(page_size),
        _I(1 if write_kv else 0), _stream()), "rope_kv_write_partial")


def rope_kv_write(qkv: torch.Tensor, H: int, G: int, d: int, rotary_dim: int, pairing: int,
                  cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                  kv: Optional[torch.Tensor], slot_map: Optional[torch.Tensor], page_size: int,
                  write_kv: bool) -> None:
    """Rotate q and k of qkv [T, (H+2G)*d] in place by the table rows of ``positions`` and
    write k, v to their slots of ``kv`` [pages, 2, G, page_size, d]."""
    T = qkv.shape[0]
    assert qkv.shape[1] == (H + 2 * G) * d and positions.dtype == torch.int32
    _contig(qkv, "qkv")
    if cos is not None:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] == rotary_dim // 2
    if write_kv:
        assert kv is not None and kv.dtype == qkv.dtype and slot_map.dtype == torch.int32
        assert tuple(kv.shape[1:]) == (2, G, page_size, d), (kv.shape, G, page_size, d)
        _contig(kv, "kv")
    _check(library("elementwise").qd_rope_kv_write(
        _ptr(qkv), _I(dtype_code(qkv.dtype)), _I(T), _I(H), _I(G), _I(d), _I(rotary_dim), _I(pairing),
        _ptr(cos), _ptr(sin), _ptr(positions), _ptr(kv), _ptr(slot_map), _I(page_size),
        _I(1 if write_kv else 0), _stream()), "rope_kv_write")


def rope_kv_write_biased(qkv: torch.Tensor, bias: Optional[torch.Tensor], H: int, G: int, d: int, rotary_dim: int,
                         pairing: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                         positions: torch.Tensor, kv: Optional[torch.Tensor], slot_map: Optional[torch.Tensor],
                         page_size: int, write_kv: bool) -> None:
    """``rope_kv_write`` with the projection's float32 bias [(H+2G)*d] added first (rounded to bfloat16 before
    the rotation); bfloat16 and the vectorized kernel's sizes only (KernelError otherwise)."""
    T = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.shape[1] == (H + 2 * G) * d and positions.dtype == torch.int32
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == (H + 2 * G) * d)
    _contig(qkv, "qkv")
    if write_kv:
        assert kv is not None and kv.dtype == qkv.dtype and tuple(kv.shape[1:]) == (2, G, page_size, d)
        _contig(kv, "kv")
    _check(library("elementwise").qd_rope_kv_write_biased(
        _ptr(qkv), _ptr(bias), _I(T), _I(H), _I(G), _I(d), _I(rotary_dim), _I(pairing), _ptr(cos), _ptr(sin),
        _ptr(positions), _ptr(kv), _ptr(slot_map), _I(page_size), _I(1 if write_kv else 0), _stream()),
        "rope_kv_write_biased")


def elementwise_plain_next() -> None:
    """The next launch of the elementwise library (the norm or the addition that takes a branch's output) is
    ordered after all earlier work of the stream, without programmatic dependent launch: for the reader of a
    batched library product."""
    fn = library("elementwise").qd_elementwise_plain_next
    fn.restype = None
    fn()


def swiglu_partial(part: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, f] = silu(sum_p part[p, t, f]) * (sum_p part[p, t, F + f]) from the float32 partial sums
    [n_parts, T, 2F] of a split-K gate/up product; out bfloat16."""
    T, F = out.shape
    assert part.dim() == 3 and tuple(part.shape[1:]) == (T, 2 * F) and part.dtype == torch.float32
    assert out.dtype == torch.bfloat16 and F % 4 == 0
    _contig(part, "part"); _contig(out, "out")
    _check(library("elementwise").qd_swiglu_partial(_ptr(part), _I(part.shape[0]), _ptr(out), _I(T), _I(F), _stream()),
           "swiglu_partial")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, f] = silu(gate_up[t, f]) * gate_up[t, F + f]."""
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F) and gate_up.dtype == out.dtype
    _contig(gate_up, "gate_up"); _contig(out, "out")
    _check(library("elementwise").qd_swiglu(_ptr(gate_up), _ptr(out), _I(dtype_code(out.dtype)), _I(T),
                                            _I(F), _stream()), "swiglu")


# ------------------------------------------------------------------------ gemm
def gemm_generic(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[T, N] = x[T, K] @ w[N, K]^T (+ bias), float32 FMA; x and out may be row-strided."""
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (T, N) and x.dtype == w.dtype
    assert x.stride(1) == 1 and out.stride(1) == 1
    _contig(w, "w")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    _check(library("gemm_generic").qd_gemm_generic(
        _ptr(x), _ptr(w), _I(dtype_code(x.dtype)), _ptr(bias), _ptr(out), _I(dtype_code(out.dtype)),
        _I(T), _I(N), _I(K), _LL(x.stride(0)), _LL(out.stride(0)), _stream()), "gemm_generic")


SKINNY_MAX_TOKENS = 64      # what the mma.sync few-token kernels take
# Who takes a product of T tokens was settled by measurement in whole decode steps (profiles/); the numbers are
# module attributes so that a measurement can move them, not switches of the environment.
SKINNY_POLICY_TOKENS = 16      # up to here the few-token kernels are the faster choice
STREAM_POLICY_TOKENS = 8       # up to here the streaming kernel takes every product
STREAM_RESIDENT_TOKENS = 16    # from there up to here it still takes a product whose result is partial sums over
# shares of K of one stage (1,024) each: the tokens' rows for such a share stay in shared memory as whole rows do
# for up to 8 tokens (a decode step at batch 16: 2.47 -> 2.13 ms at the 3B sizes, 5.33 -> 3.56 ms at the 7B sizes);
# the other products of 9 to 16 tokens (whole sums: the output projection over the vocabulary) take the
# register-load kernel
STREAM_RESIDENT_MAX_SHARES = 32
TC5_POLICY_TOKENS = 16         # from SKINNY_POLICY_TOKENS up to here the tcgen05 kernel; 16 = never:
# on row-major weights it reads 128-byte pieces of 128 rows per copy and stays below the library product
EPI_STORE, EPI_PARTIAL, EPI_SWIGLU = 0, 1, 2


def few_token_impl(T: int) -> str:
    """Which kernel takes a product of T tokens: "stream" / "regs" (mma.sync weight streamers), "tc5"
    (tcgen05 + TMA), or "" (none of the few-token kernels: the caller takes the library product)."""
    if skinny_impl == "tc5":
        return "tc5" if T <= max(TC5_POLICY_TOKENS, SKINNY_POLICY_TOKENS) else ""
    if T <= SKINNY_POLICY_TOKENS:
        # the streaming kernel is the faster one up to 8 tokens (one 8-token tile per row block); with two
        # tiles its stages shrink and the register-load kernel wins clearly (measured in whole decode steps)
        return "regs" if skinny_impl == "stream" and T > STREAM_POLICY_TOKENS else skinny_impl
    return "tc5" if T <= TC5_POLICY_TOKENS else ""


def stream_resident_shares(T: int, K: int) -> int:
    """For 9 to ``STREAM_RESIDENT_TOKENS`` tokens: the number of shares of K (one stage of the streamer each) with
    which the streaming kernel keeps the tokens resident, or 0 if this product is not taken that way."""
    if skinny_impl != "stream" or not (STREAM_POLICY_TOKENS < T <= min(16, STREAM_RESIDENT_TOKENS)):
        return 0
    chunks = (K + 1023) // 1024
    return chunks if chunks <= STREAM_RESIDENT_MAX_SHARES else 0


SWIGLU_FROM_SHARES_WIDE = True     # up to 8 tokens and a hidden size above two stages: gate/up as partial sums


def swiglu_shares(T: int, K: int, N: int) -> int:
    """The shares of K over which the stacked gate/up product [N, K] of T tokens leaves partial sums for
    ``swiglu_partial``, or 0 where the product's own SwiGLU epilogue is the better choice.  Partial sums pay
    where they keep the tokens' rows resident in the streamer: for 9 to 16 tokens, and for up to 8 tokens when
    K is wider than the rows the streamer keeps (the one-kernel form then copies the tokens with every stage)."""
    shares = stream_resident_shares(T, K)
    if shares:
        return shares
    chunks = (K + 1023) // 1024
    if SWIGLU_FROM_SHARES_WIDE and few_token_impl(T) == "stream" and T <= STREAM_POLICY_TOKENS and chunks > 2:
        sp = skinny_splits(N, K, T)
        if max(chunks * (i + 1) // sp - chunks * i // sp for i in range(sp)) <= 2:
            return sp
    return 0


def _impl_for(T: int, K: int, splits: int, epi: int) -> str:
    """The kernel one product runs on: ``few_token_impl`` by the number of tokens, and the streaming kernel for
    partial sums of 9 to 16 tokens over shares that keep the tokens resident."""
    impl = few_token_impl(T) or "tc5"
    if impl == "regs" and epi == EPI_PARTIAL and splits == stream_resident_shares(T, K):
        return "stream"
    return impl


def skinny_supported(x: torch.Tensor, w: torch.Tensor, limit: Optional[int] = None) -> bool:
    if limit is None:
        limit = max(TC5_POLICY_TOKENS, SKINNY_POLICY_TOKENS)
        if not few_token_impl(x.shape[0]):
            return False
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= limit
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_splits(N: int, K: int, T: int = 1, target_ctas: Optional[int] = None) -> int:
    """Shares of K over the grid: enough CTAs (16 rows of W each) for four per SM, every warp at
    least one group of 128 k.  The tcgen05 kernel has tiles of 128 rows and one CTA per SM."""
    impl = few_token_impl(T) or "tc5"
    if impl == "regs" and stream_resident_shares(T, K):
        return stream_resident_shares(T, K)
    if target_ctas is None:
        target_ctas = 4 * sm_count()
    if impl == "tc5":
        tiles = (N + 127) // 128
        return max(1, min((tc5_max_ctas() + tiles - 1) // tiles, ((K + 63) // 64) // 8, 16))
    tiles = (N + 15) // 16
    if impl == "stream":
        chunks = (K + 1023) // 1024          # the streaming kernel splits K in whole stages of 1024
        if T <= 8 and chunks > 2:
            # The kernel keeps the tokens in shared memory when no share of K is wider than two stages, and
            # a CTA then keeps one share for the whole launch: among the splits that allow it, take the one
            # whose busiest CTA reads least (rounds over the tiles x stages per share).
            best = None
            for sp in range((chunks + 1) // 2, min(chunks, 16) + 1):
                per_share = max(1, min(stream_max_ctas() // sp, tiles))
                widest = max(chunks * (i + 1) // sp - chunks * i // sp for i in range(sp))
                if widest > 2:
                    continue
                cost = -(-tiles // per_share) * widest
                if best is None or cost < best[0]:
                    best = (cost, sp)
            if best is not None:
                return best[1]
        return max(1, min((target_ctas + tiles - 1) // tiles, chunks, 16))
    groups = (K + 127) // 128
    return max(1, min((target_ctas + tiles - 1) // tiles, groups // 4, 16))


# Which few-token kernel runs: "stream" (persistent CTAs fed by bulk asynchronous copies,
# csrc/gemm_stream.cu) or "regs" (one wave of CTAs loading straight into registers, csrc/gemm_skinny.cu).
skinny_impl = "stream"
_FFN_FUSED = _os.environ.get("QD_FFN_FUSED", "1") != "0"      # gate/up and down of up to 8 tokens in one launch

_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the (current) CUDA device: what grids of persistent CTAs and the splits of the
    attention kernels are sized by."""
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return n


def stream_max_ctas() -> int:
    """Two persistent CTAs of the weight streamer on every multiprocessor."""
    return 2 * sm_count()


def tc5_max_ctas() -> int:
    """The tcgen05 product runs one persistent CTA per multiprocessor."""
    return sm_count()


def tile_weight(w: torch.Tensor, halves: int = 1) -> torch.Tensor:
    """W [N, K] bfloat16 -> [ceil(N/128) * ceil(K/64), 128, 64], zero-padded, each tile stored as the
    shared-memory image the tensor cores read (rows of 128 bytes; the 16-byte piece c of row r sits at
    piece c ^ (r % 8): the 128-byte swizzle): ``gemm_tc5`` fetches a tile with one contiguous 16 KB copy.
    ``halves`` = 2 tiles the gate and the up half of a stacked [2F, K] matrix separately (gate tiles
    first), as the SwiGLU epilogue wants them."""
    N, K = w.shape
    parts = w.chunk(halves, dim=0)
    out = []
    for part in parts:
        n = part.shape[0]
        nt, kt = (n + 127) // 128, (K + 63) // 64
        padded = torch.zeros((nt * 128, kt * 64), dtype=w.dtype, device=w.device)
        padded[:n, :K] = part
        tiles = padded.view(nt, 128, kt, 64).permute(0, 2, 1, 3).contiguous().view(nt * kt, 128, 8, 8)
        r = torch.arange(128, device=w.device).view(128, 1)
        c = torch.arange(8, device=w.device).view(1, 8)
        src = (c ^ (r & 7)).view(1, 128, 8, 1).expand(tiles.shape[0], 128, 8, 8)    # piece at position p holds piece p ^ (r % 8)
        out.append(torch.gather(tiles, 2, src).view(nt * kt, 128, 64))
    return torch.cat(out, dim=0).contiguous()


def gemm_tc5_status() -> int:
    """0 unless a bounded wait inside the tcgen05 kernel ran out on the current device."""
    return int(library("gemm_tc5").qd_gemm_tc5_status())


def _skinny_call(x, w, bias, out, part, T, N, K, splits, epi, what, w_tiled=False):
    out_code = dtype_code(out.dtype) if out is not None else F32
    ldo = out.stride(0) if out is not None else 0
    impl = _impl_for(T, K, splits, epi)
    if impl == "tc5":
        _check(library("gemm_tc5").qd_gemm_tc5(
            _ptr(w), _ptr(x), _LL(x.stride(0)), _ptr(bias), _ptr(out), _I(out_code), _LL(ldo), _ptr(part),
            _I(T), _I(N), _I(K), _I(splits), _I(epi), _I(tc5_max_ctas()), _I(1 if w_tiled else 0), _stream()), what)
    elif impl == "stream":
        _check(library("gemm_stream").qd_gemm_stream(
            _ptr(w), _ptr(x), _LL(x.stride(0)), _ptr(bias), _ptr(out), _I(out_code), _LL(ldo), _ptr(part),
            _I(T), _I(N), _I(K), _I(splits), _I(epi), _I(stream_max_ctas()), _stream()), what)
    else:
        _check(library("gemm_skinny").qd_gemm_skinny(
            _ptr(w), _ptr(x), _LL(x.stride(0)), _ptr(bias), _ptr(out), _I(out_code), _LL(ldo), _ptr(part),
            _I(T), _I(N), _I(K), _I(splits), _I(epi), _stream()), what)


def gemm_stream_status() -> int:
    """0 unless a bounded wait inside the streaming kernel ran out on the current device."""
    return int(library("gemm_stream").qd_gemm_stream_status())


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[T, N] = x @ w^T (+ bias) for T <= 64, bfloat16 in, out bfloat16 or float32."""
    T, K = x.shape
    N = w.shape[0]
    assert skinny_supported(x, w, 1 << 30) and out.shape == (T, N) and out.stride(1) == 1
    _contig(w, "w")
    _skinny_call(x, w, bias, out, None, T, N, K, 1, EPI_STORE, "gemm_skinny")


def gemm_skinny_partial(x: torch.Tensor, w: torch.Tensor, splits: int) -> torch.Tensor:
    """float32 partial sums [splits, T, N] of x @ w^T over ``splits`` shares of K."""
    T, K = x.shape
    N = w.shape[0]
    assert skinny_supported(x, w, 1 << 30)
    _contig(w, "w")
    part = torch.empty((splits, T, N), dtype=torch.float32, device=x.device)
    _skinny_call(x, w, None, None, part, T, N, K, splits, EPI_PARTIAL, "gemm_skinny_partial")
    return part


def gemm_skinny_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, F] = silu(x @ Wg^T) * (x @ Wu^T) with w_gate_up = [Wg; Wu] of shape [2F, K]."""
    T, K = x.shape
    N = w_gate_up.shape[0]
    assert skinny_supported(x, w_gate_up, 1 << 30) and out.shape == (T, N // 2) and out.dtype == torch.bfloat16
    _contig(w_gate_up, "w"); _contig(out, "out")
    _skinny_call(x, w_gate_up, None, out, None, T, N, K, 1, EPI_SWIGLU, "gemm_skinny_swiglu")


def ffn_stream_supported(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Whether the one-launch feed-forward (gate/up + SwiGLU, a wait between CTAs, down) takes these sizes."""
    T, D = x.shape
    F = w_down.shape[1]
    return (_FFN_FUSED and T <= 8 and D <= 2048 and few_token_impl(T) == "stream" and skinny_supported(x, w_gate_up)
            and w_down.dtype == torch.bfloat16 and F % 8 == 0 and w_gate_up.shape[0] == 2 * F
            and w_down.shape[0] == D)


FFN_SYNC_WORDS = 64      # words of device memory a layer's one-launch feed-forward synchronises through


def ffn_stream(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, barrier: torch.Tensor,
               timeline: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 partial sums [splits, T, D] of (silu(x Wg^T) * (x Wu^T)) Wd^T for up to 8 tokens, in one
    launch of the weight streamer: between the two products a CTA waits for the others' columns of h that its
    share of the second product reads, its producer warp meanwhile fetches the second product's first weights.  ``barrier``: ``FFN_SYNC_WORDS`` int32 words
    on the device, zero before their first use, that belong to the caller (no two launches that may run
    at the same time share them); every launch leaves them ready for the next.  ``timeline``: for measurements,
    int64 [CTAs, 8] that takes the kernel's own nanosecond stamps."""
    assert barrier.dtype == torch.int32 and barrier.numel() >= FFN_SYNC_WORDS and barrier.is_cuda
    T, D = x.shape
    F = w_down.shape[1]
    _contig(w_gate_up, "w_gate_up"); _contig(w_down, "w_down")
    splits = skinny_splits(D, F, T)
    h = torch.empty((T, F), dtype=torch.bfloat16, device=x.device)
    part = torch.empty((splits, T, D), dtype=torch.float32, device=x.device)
    _check(library("gemm_stream").qd_ffn_stream(
        _ptr(w_gate_up), _ptr(x), _LL(x.stride(0)), _ptr(h), _LL(h.stride(0)), _ptr(w_down), _ptr(part), _I(T), _I(D),
        _I(F), _I(splits), _ptr(barrier), _I(stream_max_ctas()), _ptr(timeline), _stream()), "ffn_stream")
    return part


# ------------------------------------------------------------------- attention
def paged_attention_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                            block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                            n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float,
                            window: int) -> None:
    """Attention of every token over keys 0..pos (or the last ``window`` of them) of its request,
    read from ``kv`` [pages, 2, G, page_size, d] through ``block_table`` [R, max_blocks].
    ``q`` points at the first query element; rows are ``q_stride`` elements apart."""
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert token_req.dtype == torch.int32 and positions.dtype == torch.int32
    assert out.shape == (n_tokens, H * d) and kv.dtype == q.dtype == out.dtype
    assert tuple(kv.shape[1:]) == (2, G, page_size, d)
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_generic").qd_paged_attention_generic(
        _ptr(q), _LL(q_stride), _ptr(out), _LL(out.stride(0)), _ptr(kv), _I(dtype_code(q.dtype)),
        _ptr(block_table), _I(block_table.shape[1]), _ptr(token_req), _ptr(positions), _I(n_tokens),
        _I(H), _I(G), _I(d), _I(page_size), _F(scale), _I(window), _stream()), "paged_attention_generic")


FLASH_HEAD_DIMS = (16, 32, 48, 64, 96, 128)


def flash_decode_supported(dtype, H: int, G: int, d: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and d in FLASH_HEAD_DIMS and H // G <= 16 and page_size % 16 == 0


def flash_prefill_supported(dtype, H: int, G: int, d: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and d in FLASH_HEAD_DIMS and H // G <= 64


_TICKETS = 1 << 16
_tickets = {}
# split-KV decode attention fed by TMA tensor copies at head sizes 64 and 128 (batch 64 at context 2,176: 43.0
# against 47.1 us a launch; QD_DECODE_TMA=0 keeps the cp.async kernel)
_DECODE_TMA = _os.environ.get("QD_DECODE_TMA", "1") != "0"


def decode_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                     block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                     n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float, window: int,
                     splits: int, fused_combine: bool = True) -> None:
    """One query token per request over its cached keys (tensor cores, keys split over ``splits``
    CTAs per (request, kv head); partial results go through scratch memory when splits > 1)."""
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert out.shape == (n_tokens, H * d) and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    part_o = part_ml = tickets = None
    if splits > 1:
        part_o = torch.empty((n_tokens * H * splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_tokens * H * splits, 2), dtype=torch.float32, device=q.device)
        if fused_combine and n_tokens * G <= _TICKETS:
            tickets = _tickets.get(q.device)
            if tickets is None:     # zero once; every launch leaves them zero again
                tickets = _tickets[q.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=q.device)
    if _DECODE_TMA and d in (64, 128) and splits <= 64 and (splits == 1 or tickets is not None):
        # K/V chunks by TMA tensor copies instead of 16-byte cp.async
        _check(library("attention_flash").qd_decode_attention_tma(
            _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _LL(kv.shape[0]), _ptr(block_table),
            _I(block_table.shape[1]), _ptr(token_req), _ptr(positions), _I(n_tokens), _I(H), _I(G), _I(d),
            _I(page_size), _F(scale), _I(window), _I(splits), _ptr(part_o), _ptr(part_ml), _ptr(tickets),
            _stream()), "decode_attention_tma")
        return
    _check(library("attention_flash").qd_decode_attention(
        _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(token_req), _ptr(positions), _I(n_tokens), _I(H), _I(G), _I(d), _I(page_size), _F(scale),
        _I(window), _I(splits), _ptr(part_o), _ptr(part_ml), _ptr(tickets), _stream()), "decode_attention")


def decode_rope_supported(dtype: torch.dtype, H: int, G: int, d: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and d in (16, 32, 48, 64, 96, 128) and H % G == 0 and H // G <= 16
            and page_size % 16 == 0)


def decode_attention_rope(part: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, kv: torch.Tensor,
                          block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                          slot_map: torch.Tensor, H: int, G: int, d: int, page_size: int, scale: float,
                          window: int, splits: int, write_kv: bool, rotary_dim: int, pairing: int,
                          cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                          timeline: Optional[torch.Tensor] = None) -> None:
    """One decoded token per request, from the float32 partial sums part [n_parts, T, (H+2G)*d] of q, k, v:
    bias, rotation by position, cache write and attention over the paged cache in one launch; the splits
    of a (token, kv head) combine through scratch memory, the last CTA to finish doing the sum."""
    n_parts, T, W = part.shape
    assert part.dtype == torch.float32 and W == (H + 2 * G) * d and out.shape == (T, H * d)
    assert out.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and positions.dtype == torch.int32
    _contig(part, "part"); _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == W
    part_o = part_ml = tickets = None
    if splits > 1:
        if T * G > _TICKETS:
            raise KernelError("decode_attention_rope: more (token, kv head) pairs than tickets")
        part_o = torch.empty((T * H * splits, d), dtype=torch.float32, device=part.device)
        part_ml = torch.empty((T * H * splits, 2), dtype=torch.float32, device=part.device)
        tickets = _tickets.get(part.device)
        if tickets is None:     # zero once; every launch leaves them zero again
            tickets = _tickets[part.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=part.device)
    _check(library("attention_decode_rope").qd_decode_attention_rope(
        _ptr(part), _I(n_parts), _ptr(bias), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(token_req), _ptr(positions), _ptr(slot_map), _I(T), _I(H), _I(G), _I(d), _I(page_size), _F(scale),
        _I(window), _I(splits), _I(1 if write_kv else 0), _ptr(cos), _ptr(sin), _I(rotary_dim), _I(pairing),
        _ptr(part_o), _ptr(part_ml), _ptr(tickets), _ptr(timeline), _stream()),
        "decode_attention_rope")


def prefill_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                      block_table: torch.Tensor, cu_tokens: torch.Tensor, start_pos: torch.Tensor,
                      n_requests: int, n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float,
                      window: int) -> None:
    """Portions of ``n_requests`` requests (tokens cu_tokens[r]..cu_tokens[r+1]-1 at positions
    start_pos[r]..) over their cached keys, causal, on tensor cores."""
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    # cu_tokens holds rows of q and out: they may start past row 0 (the rows before belong to another kernel)
    assert out.shape[0] >= n_tokens and out.shape[1] == H * d and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.shape[0] >= n_requests
    assert cu_tokens.dtype == torch.int32 and start_pos.dtype == torch.int32
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_flash").qd_prefill_attention(
        _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(cu_tokens), _ptr(start_pos), _I(n_requests), _I(n_tokens), _I(H), _I(G), _I(d), _I(page_size),
        _F(scale), _I(window), _stream()), "prefill_attention")


# -------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, draws: torch.Tensor,
           out: torch.Tensor) -> None:
    """out[r] = sampled token of logits[r] (float32 [R, V]); temperature 0 is argmax."""
    R, V = logits.shape
    assert logits.dtype == torch.float32 and temperature.dtype == torch.float32
    assert top_k.dtype == torch.int32 and draws.dtype == torch.float32 and out.dtype == torch.int32
    _contig(logits, "logits")
    _check(library("sampling").qd_sample(_ptr(logits), _I(R), _I(V), _ptr(temperature), _ptr(top_k),
                                         _ptr(draws), _ptr(out), _stream()), "sample")


def prefill_tc5_supported(dtype, H: int, G: int, d: int, page_size: int) -> bool:
    """What the tcgen05 prefill attention takes: bfloat16, head size 64 or 128, up to 16 query heads per KV
    head, pages of a multiple of 16 tokens."""
    return (dtype == torch.bfloat16 and d in (64, 128) and H % G == 0 and 1 <= H // G <= 16
            and page_size % 16 == 0)


def prefill_attention_tc5(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                          block_table: torch.Tensor, cu_tokens: torch.Tensor, start_pos: torch.Tensor,
                          n_requests: int, n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float,
                          window: int, timeline: Optional[torch.Tensor] = None) -> None:
    """``prefill_attention`` on tcgen05 tensor cores (accumulators in tensor memory, K/V tiles by TMA)."""
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert out.shape[0] >= n_tokens and out.shape[1] == H * d and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.shape[0] >= n_requests
    assert cu_tokens.dtype == torch.int32 and start_pos.dtype == torch.int32
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_tc5").qd_prefill_attention_tc5(
        _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _LL(kv.shape[0]), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(cu_tokens), _ptr(start_pos), _I(n_requests), _I(n_tokens), _I(H), _I(G), _I(d), _I(page_size),
        _F(scale), _I(window), _ptr(timeline), _stream()), "prefill_attention_tc5")


def prefill_attention_tc5_status() -> int:
    """0, or which bounded wait of the tcgen05 attention kernel ran out since the last call (synchronises)."""
    return int(library("attention_tc5").qd_prefill_attention_tc5_status())


# library -> (its status function, its wait probe): the kernels with bounded waits on mbarriers or a grid barrier
_STATUS = {"gemm_stream": ("qd_gemm_stream_status", "qd_gemm_stream_wait_probe"),
           "gemm_tc5": ("qd_gemm_tc5_status", "qd_gemm_tc5_wait_probe"),
           "attention_tc5": ("qd_prefill_attention_tc5_status", "qd_prefill_attention_tc5_wait_probe"),
           "attention_flash": ("qd_decode_attention_tma_status", "qd_decode_attention_tma_wait_probe")}


def check_status() -> None:
    """Raise if a bounded wait inside one of the kernels with mbarrier or grid-barrier waits ran out since the
    last call: the results of that launch were void.  Synchronises the device; asks only the libraries this
    process has loaded; a status is reported once."""
    bad = []
    for name, (fn, _) in _STATUS.items():
        if _library_loaded(name):
            code = int(getattr(library(name), fn)())
            if code != 0:
                bad.append(f"{name} (status {code})")
    if bad:
        raise KernelError("a bounded wait ran out inside a kernel of " + ", ".join(bad) +
                          "; results of launches since the last check are invalid")


def wait_probe(name: str, poll_limit: int = 2048) -> None:
    """Launch library ``name``'s probe: one warp waits ``poll_limit`` polls, through the library's own wait
    function, on an mbarrier that nobody arrives at.  The wait runs out, the kernel ends, and the next
    ``check_status`` raises.  For tests of that chain; it harms nothing else."""
    _check(getattr(library(name), _STATUS[name][1])(ctypes.c_uint(poll_limit), _stream()), f"{name} wait probe")


# ------------------------------------------------------------------ the layers of a prompt step from native code
class PromptLayer(ctypes.Structure):
    """One schedule entry of the native prompt step (PeLayer in csrc/prompt_exec.cu)."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("norm1_w", "norm2_w", "wqkv", "bqkv", "wo", "wgu", "wd", "kv")] + \
        [("eps1", ctypes.c_float), ("eps2", ctypes.c_float), ("write_kv", ctypes.c_int), ("pad", ctypes.c_int)]


class PromptFns(ctypes.Structure):
    """Addresses of the launchers and of the library product that the native prompt step calls."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("add_rmsnorm", "rope_kv_write", "swiglu", "attention_regs",
                                               "attention_tc5", "attention_decode", "gemm_ex", "blas",
                                               "gemm_batched", "plain_next")]


class PromptParams(ctypes.Structure):
    """Arguments of the native prompt step (PeParams in csrc/prompt_exec.cu)."""
    _fields_ = [("fn", PromptFns), ("layers", ctypes.c_void_p), ("n_layers", ctypes.c_int)] + \
        [(n, ctypes.c_int) for n in ("T", "R", "D", "H", "G", "d", "F", "page_size", "window", "rotary_dim",
                                     "pairing", "max_blocks", "use_tc5", "n_wanted")] + \
        [("scale", ctypes.c_float), ("final_eps", ctypes.c_float), ("n_pages", ctypes.c_longlong)] + \
        [(n, ctypes.c_void_p) for n in ("positions", "slot_map", "block_table", "cu_tokens", "start_pos",
                                        "logit_rows", "cos_t", "sin_t", "final_w", "x", "delta0", "h", "qkv",
                                        "attn", "delta", "gu", "act", "hrows")] + \
        [("n_decode", ctypes.c_int), ("decode_splits", ctypes.c_int)] + \
        [(n, ctypes.c_void_p) for n in ("token_req", "part_o", "part_ml", "tickets", "down_part")] + \
        [("down_shares", ctypes.c_int), ("pad2", ctypes.c_int)]


def prompt_exec_struct_sizes_match() -> bool:
    a, b = ctypes.c_int(0), ctypes.c_int(0)
    library("prompt_exec").qd_prompt_exec_struct_sizes(ctypes.byref(a), ctypes.byref(b))
    return a.value == ctypes.sizeof(PromptLayer) and b.value == ctypes.sizeof(PromptParams)


def _loaded_cublas() -> ctypes.CDLL:
    """The cuBLAS that this process has loaded already (torch's), found among the mapped files: the native
    prompt step must call the same copy whose handle it is given."""
    torch.cuda.current_blas_handle()          # makes torch load and initialise it
    with open("/proc/self/maps") as f:
        for line in f:
            path = line.split(None, 5)[-1].strip() if line.count("/") else ""
            if "/libcublas.so" in path:
                return ctypes.CDLL(path)
    raise KernelError("no libcublas is loaded in this process")


_prompt_fns: dict = {}


def prompt_fns(use_tc5: bool, with_decode: bool = False) -> PromptFns:
    """The launchers' addresses (their libraries are built and loaded on the first call; an attention
    kernel that the model does not use stays unbuilt); ``blas`` is filled in per step."""
    fns = _prompt_fns.get((use_tc5, with_decode))
    if fns is None:
        addr = lambda f: ctypes.cast(f, ctypes.c_void_p).value
        ew = library("elementwise")
        fns = PromptFns()
        fns.add_rmsnorm = addr(ew.qd_add_rmsnorm)
        fns.rope_kv_write = addr(ew.qd_rope_kv_write_biased)
        fns.swiglu = addr(ew.qd_swiglu)
        if use_tc5:
            fns.attention_tc5 = addr(library("attention_tc5").qd_prefill_attention_tc5)
        else:
            fns.attention_regs = addr(library("attention_flash").qd_prefill_attention)
        if with_decode:
            fns.attention_decode = addr(library("attention_flash").qd_decode_attention)
        fns.gemm_ex = addr(_loaded_cublas().cublasGemmEx)
        fns.gemm_batched = addr(_loaded_cublas().cublasGemmStridedBatchedEx)
        fns.plain_next = addr(ew.qd_elementwise_plain_next)
        _prompt_fns[(use_tc5, with_decode)] = fns
    return fns


def decode_scratch(n_tokens: int, H: int, d: int, G: int, splits: int, device):
    """(part_o, part_ml, tickets) for a split-KV decode attention launch of ``n_tokens`` tokens."""
    if splits <= 1:
        return None, None, None
    part_o = torch.empty((n_tokens * H * splits, d), dtype=torch.float32, device=device)
    part_ml = torch.empty((n_tokens * H * splits, 2), dtype=torch.float32, device=device)
    tickets = None
    if n_tokens * G <= _TICKETS:
        tickets = _tickets.get(device)
        if tickets is None:     # zero once; every launch leaves them zero again
            tickets = _tickets[device] = torch.zeros(_TICKETS, dtype=torch.int32, device=device)
    return part_o, part_ml, tickets


def prompt_exec(params: PromptParams, n_launches: int) -> None:
    """All layers of a prompt step and the final norm at the wanted rows, launched from one native loop on
    the step's stream (``params.fn.blas`` must be a cuBLAS handle bound to that stream)."""
    stream = _stream()
    _launch_count[0] += n_launches - 1
    code = library("prompt_exec").qd_prompt_exec(ctypes.byref(params), stream)
    if code >= 20000:
        raise KernelError(f"prompt_exec: cuBLAS status {code - 20000}")
    _check(code, "prompt_exec")

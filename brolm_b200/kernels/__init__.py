"""Python face of the hand-written CUDA kernels.

Every function takes CUDA tensors, checks what the kernel cannot check itself,
and launches on the current torch stream.  There is no CPU path and no
library fallback: a missing build or a CPU tensor raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from .build import KernelBuildError, build_all, library_loaded, load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {
    10001: "unsupported element type",
    10002: "a size the kernel does not take",
    10003: "a size beyond the kernel's limit",
    10004: "a stride or pointer that is not aligned as the kernel needs",
}
ACTIVATIONS = {"gelu_tanh": 0, "gelu_pytorch_tanh": 0, "silu": 1}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("brolm_b200 kernels run on CUDA tensors only; there is no CPU path")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


B200_SMS = 148
_sms: dict = {}


def device_sms(device=None) -> int:
    """How many SMs the device of the kernels' launches has, asked once per device.  Without a CUDA
    device (the policy functions below are plain arithmetic and are tested on the CPU) the B200's 148."""
    if not torch.cuda.is_available():
        return B200_SMS
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    n = _sms.get(index)
    if n is None:
        n = _sms[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


_launches = 0


def launch_count() -> int:
    """How many of this library's own kernels have been launched by this process."""
    return _launches


def add_launches(n: int) -> None:
    """Count kernels that ran without passing through this module (a replayed CUDA graph)."""
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[status]}")
    raise KernelError(f"{what}: CUDA error {status}")


_fn_cache: dict[str, ctypes._CFuncPtr] = {}


def _fn(lib: str, name: str, argtypes: list) -> ctypes._CFuncPtr:
    f = _fn_cache.get(name)
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[name] = f
    return f


# ---------------------------------------------------------------------------
def embed_scale(ids: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[t] = float(table[ids[t]]) * scale;  ids int32, out float32 (tokens, hidden)."""
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous()
    f = _fn("core", "brolm_embed_scale", [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _code(table), scale, _ptr(out), ids.numel(), table.shape[1], _stream()),
           "embed_scale")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * (offset + weight)."""
    assert x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n = out.shape[0]
    hidden = x.shape[-1]
    assert weight.numel() == hidden and out.shape[-1] == hidden
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    else:
        assert x.shape[0] == n
    f = _fn("core", "brolm_rmsnorm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_int,
                                      c_int, c_int, c_void_p])
    _check(f(_ptr(x), _code(x), _ptr(rows), _ptr(weight), _code(weight), eps, offset, _ptr(out), _code(out), n,
             hidden, _stream()), "rmsnorm")


def residual_rmsnorm(h: torch.Tensor, y: torch.Tensor, post_weight: Optional[torch.Tensor], post_eps: float,
                     post_offset: float, next_weight: Optional[torch.Tensor], next_eps: float, next_offset: float,
                     out: Optional[torch.Tensor]) -> None:
    """h += rmsnorm(y; post) (or y when post_weight is None); out = rmsnorm(h; next) when next_weight is given.

    ``y`` may be [parts, rows, hidden]: partial sums that are added in order first."""
    assert h.dtype == torch.float32 and h.is_contiguous() and y.is_contiguous() and tuple(y.shape[-2:]) == tuple(h.shape)
    n_parts, part_stride = (y.shape[0], y.stride(0)) if y.dim() == 3 else (1, 0)
    wd = None
    for w in (post_weight, next_weight):
        if w is not None:
            assert w.is_contiguous() and w.numel() == h.shape[-1]
            if wd is not None and w.dtype != wd:
                raise KernelError("residual_rmsnorm: both gains must have one element type")
            wd = w.dtype
    if next_weight is not None:
        assert out is not None and out.is_contiguous() and out.shape == h.shape
    f = _fn("core", "brolm_residual_rmsnorm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_float, c_float,
                                               c_void_p, c_float, c_float, c_int, c_void_p, c_int, c_int, c_int,
                                               c_void_p])
    _check(f(_ptr(h), _ptr(y), _code(y), n_parts, part_stride, _ptr(post_weight), post_eps, post_offset, _ptr(next_weight), next_eps,
             next_offset, _CODES[wd] if wd is not None else F32, _ptr(out) if next_weight is not None else None,
             _code(out) if next_weight is not None else F32, h.shape[0], h.shape[-1], _stream()),
           "residual_rmsnorm")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: Optional[torch.Tensor], n_q: int, n_kv: int,
                  head_dim: int, rotary_dim: int, k_pages: Optional[torch.Tensor] = None,
                  v_pages: Optional[torch.Tensor] = None, cache_rows: Optional[torch.Tensor] = None,
                  page_size: int = 64) -> None:
    """Rotate q and k inside qkv (tokens, (n_q + 2 n_kv) * head_dim) and write k, v into the cache pages.

    ``cache_rows[t]`` = page * page_size + place of token t, negative when the token is not kept."""
    assert qkv.is_contiguous() and qkv.shape[1] == (n_q + 2 * n_kv) * head_dim
    assert positions.dtype == torch.int32 and positions.numel() == qkv.shape[0]
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None
        assert k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim), (k_pages.shape, n_kv, page_size, head_dim)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == qkv.shape[0]
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (rotary_dim // 2, 2)
    f = _fn("core", "brolm_rope_kv_write", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                            c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), _code(qkv), _ptr(positions), _ptr(cos_sin), n_q, n_kv, head_dim, rotary_dim, _ptr(k_pages),
             _ptr(v_pages), _ptr(cache_rows) if k_pages is not None else None, page_size, qkv.shape[0], _stream()),
           "rope_kv_write")


def rope_kv_write_parts(parts: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                        cos_sin: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int,
                        k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                        cache_rows: Optional[torch.Tensor] = None, page_size: int = 64) -> None:
    """``rope_kv_write`` for a q/k/v projection that arrives as float32 partial sums of K slices,
    ``parts`` [slices, tokens, width]: the slices are added in order, q and k rotated over the whole head,
    and the result rounded once to bfloat16 into ``qkv`` (tokens, width) and into the cache pages."""
    width = (n_q + 2 * n_kv) * head_dim
    assert parts.dtype == torch.float32 and parts.dim() == 3 and parts.shape[2] == width and parts.stride(2) == 1
    assert parts.stride(1) == width and qkv.dtype == torch.bfloat16 and qkv.shape == (parts.shape[1], width)
    assert qkv.stride(1) == 1 and head_dim % 16 == 0
    assert positions.dtype == torch.int32 and positions.numel() == qkv.shape[0]
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (head_dim // 2, 2)
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None and k_pages.dtype == torch.bfloat16
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == qkv.shape[0]
    f = _fn("core", "brolm_rope_kv_write_parts", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                                  c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(parts), parts.shape[0], parts.stride(0), _ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(cos_sin),
             n_q, n_kv, head_dim, _ptr(k_pages), _ptr(v_pages), _ptr(cache_rows) if k_pages is not None else None,
             page_size, qkv.shape[0], _stream()), "rope_kv_write_parts")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = act(gate) * up for gate_up = [gate | up] (tokens, 2 * inter)."""
    assert gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype
    assert gate_up.shape[1] == 2 * out.shape[1] and gate_up.shape[0] == out.shape[0]
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation '{activation}' (known: {sorted(ACTIVATIONS)})")
    f = _fn("core", "brolm_gated_act", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _code(out), out.shape[0], out.shape[1], ACTIVATIONS[activation], _stream()),
           "gated_act")


def softcap(x: torch.Tensor, out: torch.Tensor, cap: float) -> None:
    """out (float32) = cap * tanh(x / cap); cap <= 0 only converts."""
    assert x.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32 and x.numel() == out.numel()
    f = _fn("core", "brolm_softcap", [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_ptr(x), _code(x), _ptr(out), x.numel(), cap, _stream()), "softcap")


def linear_f32(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out (M, N) = x (M, K) @ weight (N, K)^T, all float32, rows may be strided."""
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and out.dtype == torch.float32
    assert x.dim() == 2 and weight.dim() == 2 and out.dim() == 2
    assert x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and tuple(out.shape) == (M, N)
    f = _fn("linear_f32", "brolm_linear_f32", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                               c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, _stream()),
           "linear_f32")


SKINNY_MAX_ROWS = 16


def skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the few-token product kernel takes these operands."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and
            0 < x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and
            x.stride(0) % 8 == 0 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and
            x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _stream_share(fill: float) -> float:
    """Which part of the memory's rate a stream of weights reaches while an SM holds ``fill`` of the
    blocks it has room for (their weights in flight against the memory's latency): measured with the
    few-token product, 0.45 with one block of three, 0.75 with two, 0.95 with all three."""
    pts = ((0.0, 0.0), (1.0 / 3, 0.45), (2.0 / 3, 0.75), (1.0, 0.95))
    for (x0, y0), (x1, y1) in zip(pts, pts[1:]):
        if fill <= x1:
            return y0 + (y1 - y0) * (fill - x0) / (x1 - x0)
    return 0.95


def _rounds_cost(blocks: int, per_sm: int, sms: int, nbytes: float) -> float:
    """Estimated time, in bytes at the memory's full rate, of ``blocks`` equal blocks that stream ``nbytes``
    in all, ``per_sm`` of them fitting an SM at a time: round after round of blocks, each round at the
    rate its fill allows, plus 1.5 us for a round's start and end."""
    left, cost = blocks, 0.0
    while left > 0:
        now = min(left, per_sm * sms)
        cost += 1.5e-6 * 6.5e12 + nbytes * now / blocks / _stream_share(now / float(per_sm * sms))
        left -= now
    return cost


def skinny_rope_tiles(width: int, k: int, sms: Optional[int] = None) -> int:
    """16-row tiles of W per block (1 or 2) for the fused q/k/v projection, which cannot be cut along K:
    whichever fills the rounds of blocks better.  4096 rows (Gemma 2 2B): 256 blocks of one tile, three
    to an SM; 8192 rows (9B, 27B): 512 such blocks would be one round and a thin second one, 256 blocks of
    two tiles, two to an SM, are one round."""
    sms = sms or device_sms()
    tiles = (width + 15) // 16
    if tiles % 2:
        return 1
    nbytes = float(width) * k * 2.0
    return 1 if _rounds_cost(tiles, 3, sms, nbytes) <= _rounds_cost(tiles // 2, 2, sms, nbytes) else 2


def skinny_parts(x: torch.Tensor, weight: torch.Tensor, sms: Optional[int] = None) -> int:
    """Into how many slices of K a few-token product is cut.

    A block streams 16 rows of W over its slice, three blocks share an SM, and a stream runs near the
    memory's rate only while the SMs hold about three blocks each: with one block an SM reaches about
    0.45 of its share, with two 0.75, with three 0.95 (the weights of a block in flight against the
    memory's latency).  The slices decide how many blocks there are and so how full the rounds of
    blocks are; a last round of a few blocks streams slowly and is what to avoid.  The number of
    slices (at most 8, at least 8 blocks of 64 k each) with the shortest estimated time is taken; every
    slice is another float copy of the output for the kernel after it to add, which counts too.
    Measured, product + residual kernel, microseconds at 8 tokens, by slices 1 / 2 / 3 / 4:
    2304 x 9216 (2B down) 14.4 / 12.5 / 11.8 / 14.8; 4608 x 36864 (27B down) 74.0 / 72.9 / 63.2 / 67.4;
    3584 x 4096 (9B o) 10.7 / 11.8 / 12.2 / 12.0."""
    sms = sms or device_sms(x.device if x.is_cuda else None)
    blocks = (weight.shape[0] + 15) // 16
    kblocks = (x.shape[1] + 63) // 64
    nbytes = float(weight.shape[0]) * x.shape[1] * 2.0
    best, best_cost = 1, None
    for parts in range(1, 9):
        if parts > 1 and kblocks // parts < 8:
            break
        cost = _rounds_cost(blocks * parts, 3, sms, nbytes)
        cost += (parts - 1) * x.shape[0] * weight.shape[0] * 8.0 + (parts - 1) * 0.3e-6 * 6.5e12
        if best_cost is None or cost < best_cost * 0.98:
            best, best_cost = parts, cost
    return best


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
                activation: str = "gelu_tanh", cap: float = 0.0) -> None:
    """out = x @ weight^T for at most 16 rows of x (bfloat16 in, float32 accumulation).

    ``epilogue``: "store" (out bfloat16 or float32), "gated" (weight = [Wg; Wu],
    out = act(x Wg^T) * (x Wu^T)), "softcap" (out float32 = cap * tanh(. / cap)).
    """
    assert skinny_ok(x, weight) and out.stride(-1) == 1 and out.shape[-2] == x.shape[0]
    M, K = x.shape
    assert weight.shape[1] == K
    code = {"store": 0, "gated": 1, "softcap": 2}[epilogue]
    N = out.shape[-1]
    ksplit, part_stride = 1, 0
    if out.dim() == 3:                      # [parts, M, N] float32 partial sums along K
        assert code == 0 and out.dtype == torch.float32 and out.stride(1) == N
        ksplit, part_stride = out.shape[0], out.stride(0)
    assert weight.shape[0] == (2 * N if code == 1 else N)
    if code == 1:
        if activation not in ACTIVATIONS:
            raise KernelError(f"skinny_gemm: unknown activation '{activation}'")
        # a gate tile and an up tile per block, two blocks to an SM, whatever the width: blocks of four tiles (one
        # to an SM) measured slower at every size (8 tokens: 9B 40.7 against 34.5 us, 27B 109.4 against 104.6 us,
        # 2B 17.4 against 16.2 us): their last, thin round of blocks streams twice the bytes per block
        tiles = 2
    else:
        tiles = 2 if N >= 64 * device_sms(x.device) else 1
    if code == 2:
        assert out.dtype == torch.float32
    f = _fn("skinny_gemm", "brolm_skinny_gemm", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                 c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_longlong,
                                                 c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(-2), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS.get(activation, 0), cap, tiles, ksplit, part_stride,
             _stream()), "skinny_gemm")


def skinny_qkv_rope(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                    cos_sin: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int,
                    k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                    cache_rows: Optional[torch.Tensor] = None, page_size: int = 64) -> None:
    """out = x @ [Wq; Wk; Wv]^T for at most 16 rows of x, with q and k rotated over the whole head
    (pairs i, i + head_dim/2; ``cos_sin`` [positions, head_dim/2, 2], None: no rotation) and k, v written
    into the cache pages as well: ``rope_kv_write`` as the epilogue of the product, one rounding to
    bfloat16 instead of two.  Rows with a negative position are not written."""
    assert skinny_ok(x, weight) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    width = (n_q + 2 * n_kv) * head_dim
    assert weight.shape == (width, x.shape[1]) and out.shape == (x.shape[0], width) and head_dim % 16 == 0
    assert positions.dtype == torch.int32 and positions.numel() == x.shape[0]
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == head_dim // 2
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None and k_pages.dtype == torch.bfloat16
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == x.shape[0]
    f = _fn("skinny_gemm", "brolm_skinny_qkv_rope", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                                     c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), x.shape[0], x.shape[1],
             _ptr(positions), _ptr(cos_sin), n_q, n_kv, head_dim, _ptr(k_pages), _ptr(v_pages), _ptr(cache_rows),
             page_size, skinny_rope_tiles(width, x.shape[1], device_sms(x.device)), _stream()), "skinny_qkv_rope")


USE_TC_GEMM = True      # False: many-token bfloat16 products go to the library (cuBLAS) instead
USE_PAIR_GEMM = True    # False: the tcgen05 product runs one block per tile instead of a pair of SMs per tile


def gemm_tc_ok(x: torch.Tensor, weight: torch.Tensor, gated: bool = False, sms: Optional[int] = None) -> bool:
    """Whether the tcgen05 product kernel takes these operands and has enough
    128 x 256 tiles of output to put one on every SM (fewer tiles would leave
    SMs idle while the rest stream the weights)."""
    sms = sms or device_sms(x.device if x.is_cuda else None)
    out_cols = weight.shape[0] // 2 if gated else weight.shape[0]
    tiles = ((x.shape[0] + 127) // 128) * ((out_cols + (127 if gated else 255)) // (128 if gated else 256))
    return (USE_TC_GEMM and tiles >= sms and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and
            x.shape[0] > SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and
            weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and
            weight.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
            activation: str = "gelu_tanh", pairs: Optional[bool] = None) -> None:
    """out = x @ weight^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulation in tensor memory).

    Runs on pairs of SMs (``gemm_tc2``: 256 x 256 tiles, tcgen05 cta_group::2) unless ``pairs`` is False or
    ``USE_PAIR_GEMM`` is off; then one block per 128 x 256 tile.

    ``epilogue``: "store" (out bfloat16 or float32) or "gated" (weight = [Wg; Wu], out = act(x Wg^T) * (x Wu^T),
    out width a multiple of 128)."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.stride(1) == 1
    M, K = x.shape
    N = out.shape[1]
    code = {"store": 0, "gated": 1}[epilogue]
    assert weight.shape == ((2 * N if code else N), K) and out.shape[0] == M
    if activation not in ACTIVATIONS:
        raise KernelError(f"gemm_tc: unknown activation '{activation}'")
    if USE_PAIR_GEMM and pairs is not False:
        return gemm_tc2(x, weight, out, epilogue, activation)
    f = _fn("gemm_tc", "brolm_gemm_tc", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS[activation], _stream()), "gemm_tc")


def gemm_tc2(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
             activation: str = "gelu_tanh") -> None:
    """``gemm_tc`` on pairs of SMs (tcgen05 cta_group::2): 256 x 256 tiles, each block of a pair loads half
    of the weight tile.  Same operands and epilogues."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    assert weight.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == x.shape[0]
    M, K = x.shape
    code = {"store": 0, "gated": 1}[epilogue]
    N = out.shape[1]
    assert weight.shape == ((2 * N if code == 1 else N), K)
    f = _fn("gemm_tc2", "brolm_gemm_tc2", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS[activation], _stream()), "gemm_tc2")


def gemm_tc2_status(reset: bool = False) -> int:
    """0 if no bounded wait inside gemm_tc2 ever ran out; otherwise its code.  Synchronises."""
    if not library_loaded("gemm_tc2"):
        return 0
    f = load_library("gemm_tc2").brolm_gemm_tc2_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


def gemm_tc_status(reset: bool = False) -> int:
    """0 if no bounded wait inside gemm_tc (either form) ever ran out; otherwise the code of the first one.
    Synchronises."""
    pair = gemm_tc2_status(reset)
    if pair or not library_loaded("gemm_tc"):
        return pair                # (a library none of whose kernels ever ran is not built or loaded for the question)
    f = load_library("gemm_tc").brolm_gemm_tc_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


WAIT_LIBRARIES = ("gemm_tc", "gemm_tc2", "gemm_stream", "attn_tc")


def wait_control(library: str, cycles: int = 0, stall_code: int = 0) -> None:
    """The limit of the bounded waits inside one of the tcgen05 libraries, in clock cycles (0: the default of
    about a second), and, for tests of the give-up path, the code of the waits that shall behave as if
    their barrier never completed (0: none).  A wait that runs out ends its kernel early; the library's
    status function then reports the code and ``Engine.step`` raises ``StepError``."""
    if library not in WAIT_LIBRARIES:
        raise KernelError(f"wait_control: '{library}' has no bounded waits (libraries: {WAIT_LIBRARIES})")
    f = getattr(load_library(library), f"brolm_{library}_wait_control")
    f.argtypes = [c_longlong, c_int]
    f.restype = c_int
    status = f(int(cycles), int(stall_code))
    if status:
        raise KernelError(f"wait_control: CUDA error {status}")


STREAM_MAX_ROWS = 128
# Up to how many tokens the per-layer products of a step go to the tcgen05 weight stream rather than to the
# library (cuBLAS).  Measured at the Gemma 2 2B sizes, context 1280 (tokens/s, own stream against library):
# 24 rows 9,598 / 9,582; 32 rows 12,708 / 12,660; 48 rows 14,076 / 14,436; 64 rows 18,676 / 19,152;
# 96 rows 20,727 / 22,622; 128 rows 23,901 / 25,584.  With 64 and 128 token columns a stage of the ring is a
# third and a half tokens, so fewer bytes of weights are in flight per SM; up to 32 it is at least even.
# BROLM_STREAM_ROWS=128 takes every product of up to 128 tokens to the own kernel, =16 none.
STREAM_ROWS = int(os.environ.get("BROLM_STREAM_ROWS", "32"))


def stream_rows(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether a product of this many tokens is one for the tcgen05 weight stream: more rows than the
    mma.sync kernel takes (16), at most STREAM_ROWS, operands it takes."""
    return x.dim() == 2 and SKINNY_MAX_ROWS < x.shape[0] <= STREAM_ROWS and gemm_stream_ok(x, weight)


def gemm_stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tcgen05 weight-streaming product (few tokens) takes these operands."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and
            0 < x.shape[0] <= STREAM_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and
            x.stride(0) % 8 == 0 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and
            x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_stream_parts(x: torch.Tensor, weight: torch.Tensor, sms: Optional[int] = None) -> int:
    """Slices of K so that every SM gets a (128-row tile, slice) item of the weight stream."""
    sms = sms or device_sms(x.device if x.is_cuda else None)
    row_tiles = (weight.shape[0] + 127) // 128
    nkb = (x.shape[1] + 63) // 64
    want = max(1, sms // row_tiles)
    # at least a ring's worth of K blocks (8) per item: a shorter run is over before its loads are all
    # in flight, and every further slice is another float copy of the output for the reader to add
    per = max(min(8, nkb), (nkb + want - 1) // want)
    return max(1, (nkb + per - 1) // per)


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
                activation: str = "gelu_tanh", cap: float = 0.0) -> None:
    """out = x @ weight^T for at most 128 rows of x on tcgen05, the weights streamed through a TMA ring.

    ``epilogue``: "store" (out bfloat16 or float32, or [parts, M, N] float32 partial sums of K slices),
    "gated" (weight = [Wg; Wu], out = act(x Wg^T) * (x Wu^T), width a multiple of 64), "softcap" (float32)."""
    assert gemm_stream_ok(x, weight) and out.stride(-1) == 1 and out.shape[-2] == x.shape[0]
    M, K = x.shape
    code = {"store": 0, "gated": 1, "softcap": 2}[epilogue]
    N = out.shape[-1]
    assert weight.shape == ((2 * N if code == 1 else N), K)
    ksplit, part_stride = 1, 0
    if out.dim() == 3:
        assert code == 0 and out.dtype == torch.float32 and out.stride(1) == N
        ksplit, part_stride = out.shape[0], out.stride(0)
    if code == 2:
        assert out.dtype == torch.float32
    if activation not in ACTIVATIONS:
        raise KernelError(f"gemm_stream: unknown activation '{activation}'")
    f = _fn("gemm_stream", "brolm_gemm_stream", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(-2), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS[activation], cap, ksplit, part_stride, _stream()),
           "gemm_stream")


def gemm_stream_status(reset: bool = False) -> int:
    """0 if no bounded wait inside gemm_stream ever ran out; otherwise its code.  Synchronises."""
    if not library_loaded("gemm_stream"):
        return 0                   # none of its kernels ever ran: nothing is built or loaded for the question
    f = load_library("gemm_stream").brolm_gemm_stream_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


def attention_simt(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, *, n_kv: int,
                   group: int, head_dim: int, scale: float, cap: float, window: int, batch: int, max_q_len: int,
                   k: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None,
                   k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                   page_table: Optional[torch.Tensor] = None, ring: int = 0, page_size: int = 0) -> None:
    """Exact attention on CUDA cores.  Keys come from (k, v) packed like q, or from cache pages."""
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and q.dtype == out.dtype
    assert cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    kv_stride = pt_stride = 0
    if k_pages is not None:
        assert page_table is not None and page_table.dtype == torch.int32 and page_table.stride(1) == 1
        assert k_pages.dtype == q.dtype and v_pages.dtype == q.dtype and k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
        pt_stride = page_table.stride(0)
    else:
        assert k is not None and v is not None and k.dtype == q.dtype and v.dtype == q.dtype
        assert k.stride(-1) == 1 and v.stride(-1) == 1 and k.stride(0) == v.stride(0)
        kv_stride = k.stride(0)
    f = _fn("attn_simt", "brolm_attn_simt", [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p])
    _check(f(_code(q), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(kv_len), _ptr(k), _ptr(v),
             kv_stride, _ptr(k_pages), _ptr(v_pages), _ptr(page_table), pt_stride, ring, page_size, n_kv, group,
             head_dim, scale, cap, window, batch, max_q_len, _stream()), "attention_simt")


def attention_prefill_mma(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                          n_kv: int, group: int, head_dim: int, scale: float, cap: float, window: int, batch: int,
                          max_q_len: int) -> None:
    """Tensor-core attention of whole prompts that start at position 0 (bfloat16, head_dim <= 256)."""
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert k.stride(0) == v.stride(0) and cu_q.dtype == torch.int32
    f = _fn("attn_mma", "brolm_attn_prefill_mma", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int,
                                                   c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(k), _ptr(v), k.stride(0), n_kv, group,
             head_dim, scale, cap, window, batch, max_q_len, _stream()), "attention_prefill_mma")


def attention_prefill_tc_ok(head_dim: int, group: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes these sizes."""
    return head_dim in (64, 128, 256) and group > 0 and 128 % group == 0


def attention_prefill_tc_split(max_q_len: int, n_kv: int, group: int, window: int, batch: int) -> int:
    """How many of the heaviest row blocks of every (sequence, kv head) the tcgen05 prompt attention cuts in
    two along the keys (0: none): with few kv heads and a prompt of a few thousand tokens the causal blocks
    are few and of very different lengths, and halves fill the SMs better.  The launcher's own rule."""
    key = (max_q_len, n_kv, group, window, batch, torch.cuda.current_device())
    got = _split_memo.get(key)
    if got is None:
        f = _fn("attn_tc", "brolm_attn_prefill_tc_plan", [c_int, c_int, c_int, c_int, c_int])
        if len(_split_memo) > 64:
            _split_memo.clear()
        got = _split_memo[key] = int(f(max_q_len, n_kv, group, window, batch))
    return got


_split_memo: dict = {}


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                         n_kv: int, group: int, head_dim: int, scale: float, cap: float, window: int, batch: int,
                         max_q_len: int, v_lbo: int = 0, v_sbo: int = 0, n_split: Optional[int] = None) -> None:
    """tcgen05 attention of whole prompts that start at position 0 (bfloat16; head_dim 64, 128 or 256).
    ``n_split``: how many of the heaviest row blocks run as two halves of their keys, merged by the half
    that finishes second (None: ``attention_prefill_tc_split`` decides)."""
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert k.stride(0) == v.stride(0) and cu_q.dtype == torch.int32 and q.shape[0] == k.shape[0] == v.shape[0]
    if n_split is None:
        n_split = attention_prefill_tc_split(max_q_len, n_kv, group, window, batch) if PREFILL_SPLIT else 0
    part_o = part_ml = None
    if n_split > 0:
        pairs = n_split * n_kv * batch
        both = torch.empty(pairs * 2 * 128 * (head_dim + 2), dtype=torch.float32, device=q.device)
        part_o, part_ml = both[:pairs * 2 * 128 * head_dim], both[pairs * 2 * 128 * head_dim:]
    f = _fn("attn_tc", "brolm_attn_prefill_tc", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int,
                                                 c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(k), _ptr(v), k.stride(0), q.shape[0],
             n_kv, group, head_dim, scale, cap, window, batch, max_q_len, v_lbo, v_sbo, n_split, _ptr(part_o),
             _ptr(part_ml), _stream()),
           "attention_prefill_tc")


# BROLM_PREFILL_SPLIT=0: the tcgen05 prompt attention never cuts a row block's keys in two
PREFILL_SPLIT = os.environ.get("BROLM_PREFILL_SPLIT", "1") != "0"


def attention_tc_status(reset: bool = False) -> int:
    """0 if no bounded wait inside the tcgen05 attention ever ran out; otherwise its code.  Synchronises."""
    if not library_loaded("attn_tc"):
        return 0                   # none of its kernels ever ran: nothing is built or loaded for the question
    f = load_library("attn_tc").brolm_attn_tc_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


RAGGED_WAVES = int(os.environ.get("BROLM_RAGGED_WAVES", "5"))


def decode_splits(batch: int, n_kv: int, max_kv_len: int, window: int, sms: Optional[int] = None,
                  ragged: bool = False) -> int:
    """How many blocks share the keys of one (sequence, kv head): as many as make one wave of blocks
    over the SMs (a block holds an SM's shared memory alone), at least two pages per block and at
    most 40 splits (the last block's merge reads every split's partial result).
    Measured on a B200 at 8 kv-head pairs x 4: 4 splits (one wave) read 8192 keys in 54 us, 9 splits
    (two waves) in 58 us; one sequence with 4 kv heads and 8192 keys: 37 splits (148 blocks) 1.600 ms
    per decode step of the 2B sizes against 1.632 ms with 20 splits (80 blocks).

    ``ragged``: the sequences' lengths are far from equal.  One round of blocks then ends with the longest
    sequence's blocks running alone, so every sequence is cut into enough pieces for ``RAGGED_WAVES``
    rounds and the SMs even the lengths out as they take block after block.  Measured at 16 sequences of
    1,280 to 6,400 keys and 8 kv heads (128 pairs): 1 / 2 / 4 / 6 / 8 / 12 splits 147 / 128 / 118 / 114 /
    116 / 126 us; with equal lengths more than one round only costs (152 / 163 / 167 us for 1 / 2 / 4).
    (Pieces of one size for all sequences, so that a short sequence is one block and a long one many,
    were measured too: 111 to 113 us, no better than equal shares, and are not in the kernel.)"""
    sms = sms or device_sms()
    keys = min(max_kv_len, window + 63) if window > 0 else max_kv_len
    tiles = max(1, (keys + 63) // 64)
    want = max(1, sms // max(1, batch * n_kv))
    if ragged:
        want = max(want, -(-RAGGED_WAVES * sms // max(1, batch * n_kv)))
    return max(1, min(want, (tiles + 1) // 2, 40))


def attention_decode_mma(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                         k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor, *, ring: int,
                         page_size: int, n_kv: int, group: int, head_dim: int, scale: float, cap: float, window: int,
                         batch: int, n_splits: int, scratch: Optional[tuple] = None) -> None:
    """Tensor-core attention of one new token per sequence over the paged cache
    (bfloat16, head_dim <= 256, group <= 16, pages of 64 keys).  With more than
    one split the partial results go through float32 scratch: ``scratch`` =
    (part_o [batch * n_q * n_splits * head_dim], part_ml [batch * n_q * n_splits * 2]),
    made here when it is not given.  ``cu_q``, ``kv_len`` and ``page_table`` are read before the kernel
    waits for the launch before it (they are the host's description of the step, copied in before the
    step's first kernel); ``q`` and the pages are read after."""
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
    assert page_table.dtype == torch.int32 and page_table.stride(1) == 1
    assert cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    part_o = part_ml = None
    if n_splits > 1:
        n = batch * n_kv * group * n_splits
        if scratch is None:
            part_o = torch.empty(n * head_dim, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(n * 2, dtype=torch.float32, device=q.device)
        else:
            part_o, part_ml = scratch
            assert part_o.numel() >= n * head_dim and part_ml.numel() >= n * 2
    f = _fn("attn_mma", "brolm_attn_decode_mma", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                  c_float, c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(kv_len), _ptr(k_pages), _ptr(v_pages),
             _ptr(page_table), page_table.stride(0), ring, page_size, n_kv, group, head_dim, scale, cap, window,
             batch, n_splits, _ptr(part_o), _ptr(part_ml), _stream()), "attention_decode_mma")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] (int32) = first index of the maximum of logits[r] (float32)."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and out.dtype == torch.int32
    f = _fn("sampling", "brolm_argmax", [c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.shape[0], logits.shape[1], _ptr(out), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, streams: torch.Tensor,
           counter: int, out: torch.Tensor) -> None:
    """One draw per row from softmax(logits / temperature) after top-k and top-p."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert streams.dtype == torch.int32 and out.dtype == torch.int32 and streams.numel() == logits.shape[0]
    f = _fn("sampling", "brolm_sample", [c_void_p, c_int, c_int, c_float, c_int, c_float, c_ulonglong, c_void_p,
                                         c_ulonglong, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.shape[0], logits.shape[1], temperature, top_k, top_p, seed & (2 ** 64 - 1),
             _ptr(streams), counter, _ptr(out), _stream()), "sample")


__all__ = ["KernelBuildError", "KernelError", "build_all", "launch_count", "device_sms", "wait_control", "embed_scale", "rmsnorm", "residual_rmsnorm",
           "rope_kv_write", "rope_kv_write_parts", "gated_act", "softcap", "linear_f32", "skinny_gemm", "skinny_qkv_rope", "skinny_ok", "skinny_parts", "skinny_rope_tiles", "gemm_tc", "gemm_tc2", "gemm_tc2_status", "gemm_tc_ok", "gemm_tc_status", "gemm_stream", "gemm_stream_ok", "gemm_stream_parts", "stream_rows",
           "gemm_stream_status", "attention_simt", "attention_prefill_mma", "attention_prefill_tc", "attention_prefill_tc_ok", "attention_prefill_tc_split", "attention_tc_status", "attention_decode_mma",
           "decode_splits", "argmax", "sample"]

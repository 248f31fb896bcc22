"""The allocation-free decode attention, called through its exported C symbol.

Some hosts of this library may not allocate device memory once they are
running (a fixed arena owned by another runtime, a loop that bans allocator
calls).  For them ``brolm_attn_decode_mma_noalloc`` keeps the scratch of the
split-KV merge in a fixed array inside the library.  This test loads the
library with ctypes, calls the symbol itself (no Python wrapper in between)
twice in a row with different shapes, and checks each result against the
ordinary entry point, which takes its scratch from the caller, and against
the plain float64 attention (a fault that both entry points share would
pass the first comparison).  The second
call is smaller than the first, so anything stale in the shared array would
show.  It also checks that a call beyond the array's size is refused.

The file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from brolm_b200 import kernels
from brolm_b200.kernels.build import load_library
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 1 << 20          # BROLM_ATTN_NOALLOC_MAX_FLOATS in csrc/attn_decode_noalloc.h
TOL = 8e-3                    # the bfloat16 bound of tests/test_kernels_gpu.py, relative to the largest value


def symbol():
    f = load_library("attn_noalloc").brolm_attn_decode_mma_noalloc
    f.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                  c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p]
    f.restype = c_int
    return f


def case(lengths, n_q, n_kv, hd, window, seed):
    g = torch.Generator().manual_seed(seed)
    B = len(lengths)
    ring = (window + 63) // 64 * 64 if window else 1 << 30
    per = [min((n + 63) // 64, ring // 64) for n in lengths]
    pages = sum(per) + 1
    kp = torch.randn(pages, n_kv, 64, hd, generator=g).to(torch.bfloat16).to(DEV)
    vp = torch.randn(pages, n_kv, 64, hd, generator=g).to(torch.bfloat16).to(DEV)
    perm = iter(torch.randperm(pages, generator=g).tolist())
    table = torch.zeros(B, max(per), dtype=torch.int32)
    for b in range(B):
        for j in range(per[b]):
            table[b, j] = next(perm)
    q = torch.randn(B, n_q * hd, generator=g).to(torch.bfloat16).to(DEV)
    return dict(q=q, kp=kp, vp=vp, table=table.to(DEV), cu=torch.arange(B + 1, dtype=torch.int32, device=DEV),
                kv_len=torch.tensor(lengths, dtype=torch.int32, device=DEV), ring=ring, n_kv=n_kv,
                group=n_q // n_kv, hd=hd, window=window, B=B)


def run_both(f, c, splits):
    scale, cap = 1 / math.sqrt(c["hd"]), 30.0
    want = torch.empty_like(c["q"])
    kernels.attention_decode_mma(c["q"], want, c["cu"], c["kv_len"], c["kp"], c["vp"], c["table"], ring=c["ring"],
                                 page_size=64, n_kv=c["n_kv"], group=c["group"], head_dim=c["hd"], scale=scale,
                                 cap=cap, window=c["window"], batch=c["B"], n_splits=splits)
    got = torch.full_like(c["q"], 7.0)
    status = f(c["q"].data_ptr(), c["q"].stride(0), got.data_ptr(), got.stride(0), c["cu"].data_ptr(),
               c["kv_len"].data_ptr(), c["kp"].data_ptr(), c["vp"].data_ptr(), c["table"].data_ptr(),
               c["table"].stride(0), c["ring"], 64, c["n_kv"], c["group"], c["hd"], scale, cap, c["window"], c["B"],
               splits, torch.cuda.current_stream().cuda_stream)
    assert status == 0, f"brolm_attn_decode_mma_noalloc returned {status}"
    torch.cuda.synchronize()
    err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
    assert err <= TOL, f"relative error {err:.3e}"
    # and against the plain attention: each sequence's keys and values gathered back from its pages
    kp, vp, table = c["kp"].cpu(), c["vp"].cpu(), c["table"].cpu()
    n_q = c["n_kv"] * c["group"]
    for b, n in enumerate(c["kv_len"].tolist()):
        first = max(0, n - c["window"]) if c["window"] else 0
        k = torch.zeros(n, c["n_kv"] * c["hd"])
        v = torch.zeros(n, c["n_kv"] * c["hd"])
        for p in range(first, n):
            r = p % c["ring"]
            k[p] = kp[int(table[b, r // 64]), :, r % 64, :].reshape(-1).float()
            v[p] = vp[int(table[b, r // 64]), :, r % 64, :].reshape(-1).float()
        ref = plain.attention_last_query(c["q"][b].cpu().float(), k, v, n_q, c["n_kv"], c["hd"], scale, cap, c["window"])
        err = float((got[b].cpu().double() - ref).abs().max()) / float(ref.abs().max())
        assert err <= TOL, f"sequence {b}: relative error {err:.3e} against the plain attention"


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    f = symbol()
    run_both(f, case([700, 64, 1, 333, 129], n_q=8, n_kv=4, hd=256, window=0, seed=1), splits=6)
    run_both(f, case([200, 90], n_q=6, n_kv=1, hd=64, window=100, seed=2), splits=3)     # smaller: old contents remain
    run_both(f, case([65], n_q=4, n_kv=2, hd=128, window=0, seed=3), splits=1)           # no scratch at all


def test_a_call_beyond_the_fixed_scratch_is_refused():
    f = symbol()
    c = case([64] * 4, n_q=8, n_kv=4, hd=256, window=0, seed=4)
    splits = MAX_FLOATS // (c["B"] * 8 * (256 + 2)) + 1
    out = torch.full_like(c["q"], 7.0)
    status = f(c["q"].data_ptr(), c["q"].stride(0), out.data_ptr(), out.stride(0), c["cu"].data_ptr(),
               c["kv_len"].data_ptr(), c["kp"].data_ptr(), c["vp"].data_ptr(), c["table"].data_ptr(),
               c["table"].stride(0), c["ring"], 64, c["n_kv"], c["group"], c["hd"], 0.1, 0.0, 0, c["B"], splits,
               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status == 10003 and float(out.float().min()) == 7.0        # refused, nothing was launched

"""The give-up path of the bounded waits inside the tcgen05 kernels, exercised without a fault: a
library is told that the waits of one code shall never see their barrier and that the limit is a few
milliseconds; the kernel runs into the limit, gives up (its loads land, its tensor memory is freed, it
returns), the status function reports the code, ``Engine.step`` raises ``StepError``, and after the
switch is put back the same launch gives the right result.  Nothing hangs, traps or faults."""
import pytest
import torch

import brolm_b200 as bb
from brolm_b200 import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LIMIT = 8_000_000            # clock cycles: about four milliseconds


def product(fn, status, M, N, K, **kw):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    fn(x, w, out, **kw)
    torch.cuda.synchronize()
    ref = x.double().cpu() @ w.double().cpu().t()
    return out, ref


@pytest.mark.parametrize("library,code", [("gemm_stream", 3), ("gemm_tc", 3), ("gemm_tc2", 3)])
def test_a_product_whose_wait_runs_out_reports_it_and_the_next_one_is_right(library, code):
    fn = {"gemm_stream": kernels.gemm_stream, "gemm_tc": lambda x, w, o: kernels.gemm_tc(x, w, o, pairs=False),
          "gemm_tc2": kernels.gemm_tc2}[library]
    status = {"gemm_stream": kernels.gemm_stream_status, "gemm_tc": kernels.gemm_tc_status,
              "gemm_tc2": kernels.gemm_tc2_status}[library]
    M = 64 if library == "gemm_stream" else 300
    product(fn, status, M, 512, 256)                           # builds and loads the library
    assert status(reset=True) == 0
    kernels.wait_control(library, cycles=LIMIT, stall_code=code)      # code 3: the epilogue's wait for its accumulator
    try:
        product(fn, status, M, 512, 256)
        assert status(reset=False) == code
        assert status(reset=True) == code and status() == 0
    finally:
        kernels.wait_control(library, 0, 0)
    out, ref = product(fn, status, M, 512, 256)
    assert status() == 0
    assert float((out.double().cpu() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


def test_prompt_attention_whose_wait_runs_out():
    n_q, n_kv, hd, T = 4, 2, 128, 300
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, generator=g).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)

    def run():
        out = torch.empty(T, n_q * hd, dtype=torch.bfloat16, device=DEV)
        kernels.attention_prefill_tc(qkv[:, :n_q * hd], out, cu, qkv[:, n_q * hd:(n_q + n_kv) * hd],
                                     qkv[:, (n_q + n_kv) * hd:], n_kv=n_kv, group=2, head_dim=hd, scale=hd ** -0.5,
                                     cap=0.0, window=0, batch=1, max_q_len=T)
        torch.cuda.synchronize()
        return out

    good = run()
    assert kernels.attention_tc_status(reset=True) == 0
    kernels.wait_control("attn_tc", cycles=LIMIT, stall_code=8)       # code 8: the softmax warps' wait for a score tile
    try:
        run()
        assert kernels.attention_tc_status(reset=True) == 8
    finally:
        kernels.wait_control("attn_tc", 0, 0)
    again = run()
    assert kernels.attention_tc_status() == 0 and torch.equal(again, good)


def test_a_step_whose_kernel_gave_up_raises_and_the_engine_goes_on():
    """One layer of the Gemma 2 2B sizes: a prompt of 2,048 tokens runs its q/k/v product on pairs of SMs."""
    cfg = bb.Gemma2Config(vocab_size=1000, num_hidden_layers=1)
    model = bb.Model(cfg, dtype="bfloat16", device=DEV).init_random(seed=3, on_device=True)
    eng = bb.Engine(model, max_tokens=4096, max_slots=2)
    prompt = torch.randint(0, 1000, (2048,), generator=torch.Generator().manual_seed(4)).tolist()
    (s,) = eng.open(1)
    good = eng.step([s], [prompt]).clone()
    eng.close([s])
    kernels.wait_control("gemm_tc2", cycles=LIMIT, stall_code=3)
    try:
        (s,) = eng.open(1)
        with pytest.raises(bb.StepError, match="ran out"):
            eng.step([s], [prompt])
    finally:
        kernels.wait_control("gemm_tc2", 0, 0)
    eng.close([s])                                              # the slot was not committed; it goes back empty
    (s,) = eng.open(1)
    again = eng.step([s], [prompt])
    assert torch.equal(again, good)
    eng.close([s])

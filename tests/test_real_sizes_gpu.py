"""The layer sizes of the published Gemma 2 models (2B, 9B, 27B) with two layers
and a small vocabulary: the kernels must take these widths, head counts and
head sizes, and the engine must still match the plain implementation for a
prompt pass and for decode steps in a batch: in bfloat16 for all three, and in
true 32-bit for the 2B sizes (the CUDA-core product at K = 9,216 and the exact
attention at heads of 256)."""
import pytest
import torch

import brolm_b200 as bb
from tests.helpers import oracle_inputs, random_prompts
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = {
    "2b": dict(hidden_size=2304, intermediate_size=9216, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
               query_pre_attn_scalar=256, sliding_window=64),
    "9b": dict(hidden_size=3584, intermediate_size=14336, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               query_pre_attn_scalar=256, sliding_window=64),
    "27b": dict(hidden_size=4608, intermediate_size=36864, num_attention_heads=32, num_key_value_heads=16,
                head_dim=128, query_pre_attn_scalar=144, sliding_window=64),
}


@pytest.mark.parametrize("name,dtype,tol", [("2b", "bfloat16", 2e-2), ("9b", "bfloat16", 2e-2), ("27b", "bfloat16", 2e-2),
                                            ("2b", "float32", 1e-5)])
def test_layer_sizes_of_the_published_models(tmp_path, name, dtype, tol):
    cfg = bb.Gemma2Config(vocab_size=1000, num_hidden_layers=2, **SIZES[name])
    folder = str(tmp_path / name)
    # made on the device (seconds instead of minutes for 27B's 1.1 G values); the file is the same
    bb.write_random_model(cfg, folder, seed=2, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV)
    config, weights = oracle_inputs(folder)
    model = bb.load_model(folder, dtype=dtype, device=DEV)
    eng = bb.Engine(model, max_tokens=1024, max_slots=3)
    prompts = random_prompts(1000, [70, 9, 33], seed=3)
    refs = [plain.forward(config, weights, p) for p in prompts]
    pre = [66, 5, 20]
    slots = eng.open(3)
    got = eng.step(slots, [p[:k] for p, k in zip(prompts, pre)], want=[list(range(k)) for k in pre])
    off = 0
    worst = 0.0
    for r, k in zip(refs, pre):
        worst = max(worst, float((got[off:off + k].double().cpu() - r[:k]).abs().max()) / float(r[:k].abs().max()))
        off += k
    for step in range(4):
        got = eng.step(slots, [[p[k + step]] for p, k in zip(prompts, pre)])
        for i, (r, k) in enumerate(zip(refs, pre)):
            worst = max(worst, float((got[i].double().cpu() - r[k + step]).abs().max()) / float(r[k + step].abs().max()))
    eng.close(slots)
    assert worst <= tol, f"relative error {worst:.3e}"

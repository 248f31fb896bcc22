"""The choices the Python face of the kernels makes before a launch: how many
blocks share the keys of a sequence, into how many slices of K a product is
cut, which product kernel takes which operands.  Pure arithmetic on shapes;
no GPU."""
import torch

from brolm_b200 import kernels


def test_decode_splits_make_one_wave_and_keep_two_pages_a_block():
    # Gemma 2 2B: 4 kv heads, 148 SMs
    assert kernels.decode_splits(8, 4, 8192, 0) == 4                 # 8 * 4 * 4 = 128 blocks
    assert kernels.decode_splits(1, 4, 8192, 0) == 37                # 148 blocks
    assert kernels.decode_splits(64, 4, 8192, 0) == 1                # more (sequence, head) pairs than SMs
    assert kernels.decode_splits(1, 4, 200, 0) == 2                  # four pages: two a block
    assert kernels.decode_splits(1, 4, 60, 0) == 1
    assert kernels.decode_splits(1, 1, 1 << 20, 0) == 40             # never more than the merge takes cheaply
    # a window bounds the keys a sequence has, whatever its length
    assert kernels.decode_splits(1, 4, 100000, 4096) == kernels.decode_splits(1, 4, 4096 + 63, 0)
    for batch in (1, 2, 3, 8, 20):
        for n_kv in (1, 4, 16):
            s = kernels.decode_splits(batch, n_kv, 8192, 0)
            assert 1 <= s <= 40 and (s == 1 or s * batch * n_kv <= 148)
    # sequences of very unequal lengths: several rounds of blocks, so that the SMs even them out
    assert kernels.decode_splits(16, 8, 8192, 0, sms=148, ragged=True) == 6       # 768 blocks, five rounds
    assert kernels.decode_splits(16, 8, 8192, 0, sms=148) == 1
    assert kernels.decode_splits(64, 4, 300, 0, sms=148, ragged=True) == 3        # two pages a block at least
    assert kernels.decode_splits(3, 4, 8192, 0, sms=148, ragged=True) == 40


def test_slices_of_k():
    x = torch.empty(8, 9216, dtype=torch.bfloat16)
    down = torch.empty(2304, 9216, dtype=torch.bfloat16)
    gate_up = torch.empty(18432, 2304, dtype=torch.bfloat16)
    assert kernels.skinny_parts(x, down, sms=148) == 3              # 144 blocks of 16 rows: three slices are one full round (432 of 444 places)
    assert kernels.skinny_parts(torch.empty(8, 2304, dtype=torch.bfloat16), gate_up) == 1
    # 27B down: 288 blocks, three slices are nearly two full rounds; two would leave a thin second round
    assert kernels.skinny_parts(torch.empty(8, 36864, dtype=torch.bfloat16), torch.empty(4608, 36864, dtype=torch.bfloat16), sms=148) == 3
    # 9B o: 224 blocks and a short K: one slice, a second round is not worth its start
    assert kernels.skinny_parts(torch.empty(16, 4096, dtype=torch.bfloat16), torch.empty(3584, 4096, dtype=torch.bfloat16), sms=148) == 1
    assert kernels.skinny_parts(torch.empty(8, 64, dtype=torch.bfloat16), torch.empty(16, 64, dtype=torch.bfloat16)) == 1
    # the fused q/k/v projection cannot be cut along K: 16-row tiles per block by how full the rounds get
    assert kernels.skinny_rope_tiles(4096, 2304, sms=148) == 1       # 2B: 256 blocks, three to an SM
    assert kernels.skinny_rope_tiles(8192, 3584, sms=148) == 2       # 9B: 512 would be a round and a thin one; 256 of two tiles
    assert kernels.skinny_rope_tiles(48, 64, sms=148) == 1           # an odd number of tiles
    p = kernels.gemm_stream_parts(x, down)
    assert p >= 1 and p * 18 >= 100                                  # 18 row tiles: enough (tile, slice) items for the SMs


def test_which_product_takes_which_operands():
    w = torch.empty(4096, 2304, dtype=torch.bfloat16)
    few, many = torch.empty(8, 2304, dtype=torch.bfloat16), torch.empty(2048, 2304, dtype=torch.bfloat16)
    assert kernels.skinny_ok(few, w) and not kernels.skinny_ok(many, w)
    assert kernels.skinny_ok(torch.empty(16, 2304, dtype=torch.bfloat16), w)
    assert not kernels.skinny_ok(torch.empty(17, 2304, dtype=torch.bfloat16), w)
    assert not kernels.skinny_ok(few.float(), w)                      # bfloat16 only
    # the tcgen05 product wants a tile for every SM
    assert kernels.gemm_tc_ok(many, w)                                # 16 x 16 = 256 tiles
    assert not kernels.gemm_tc_ok(many, torch.empty(2304, 2304, dtype=torch.bfloat16))      # 16 x 9 = 144
    assert not kernels.gemm_tc_ok(few, w)
    assert not kernels.gemm_tc_ok(torch.empty(2048, 2308, dtype=torch.bfloat16)[:, :2301], w[:, :2301])   # K % 8
    # the weight stream takes up to 128 rows
    assert kernels.gemm_stream_ok(torch.empty(128, 2304, dtype=torch.bfloat16), w)
    assert not kernels.gemm_stream_ok(torch.empty(129, 2304, dtype=torch.bfloat16), w)
    # the tcgen05 prompt attention: head sizes 64, 128, 256 and groups that divide 128
    assert kernels.attention_prefill_tc_ok(256, 2) and kernels.attention_prefill_tc_ok(128, 8)
    assert not kernels.attention_prefill_tc_ok(80, 2) and not kernels.attention_prefill_tc_ok(128, 3)

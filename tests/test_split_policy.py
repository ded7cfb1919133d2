"""How matrix products are split over K and how prompt attention orders its blocks (host-side
policies; the SM count is given, no GPU)."""
import pytest
import torch

from rocml_b200 import kernels
from rocml_b200.parts import BuildEnv
from rocml_b200.parts import linear as L


@pytest.fixture(autouse=True)
def sms(monkeypatch):
    monkeypatch.setitem(L._SM_COUNT, 0, 148)


def product(n, k):
    lin = L.Linear(["w"], [n], k, False, BuildEnv(torch.device("cpu"), torch.bfloat16))
    return lin


# Qwen3-8B layer sizes: (name, out features, in features)
QKV, O, GATE_UP, DOWN, HEAD = (6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096)


def splits(shape, m):
    return product(*shape)._splits(m)


def test_few_rows_split_until_the_device_is_full():
    for m in (1, 8, 16):
        assert [splits(s, m) for s in (QKV, O, GATE_UP, DOWN, HEAD)] == [7, 8, 2, 16, 1]
    # 17 to 64 rows: the same counts as long as the partial sums stay below a third of the weight
    assert [splits(s, 32) for s in (QKV, O, GATE_UP, DOWN)] == [7, 8, 2, 16]
    assert [splits(s, 64) for s in (QKV, O, GATE_UP, DOWN)] == [7, 8, 2, 8]


def test_a_product_whose_tiles_fill_the_device_is_not_split_beyond_64_rows():
    assert splits(GATE_UP, 64) == 2 and splits(GATE_UP, 65) == 1 and splits(GATE_UP, 128) == 1
    assert splits(HEAD, 128) == 1
    assert [splits(s, 128) for s in (QKV, O, DOWN)] == [4, 4, 8]


def test_a_few_hundred_rows_fill_one_wave():
    # tiles of 128 rows x 256 features; splits until tiles x splits reach the multiprocessors
    assert [splits(s, 256) for s in (QKV, O, GATE_UP, DOWN)] == [3, 4, 1, 4]
    assert [splits(s, 384) for s in (QKV, O, GATE_UP, DOWN)] == [2, 3, 1, 3]
    assert [splits(s, 512) for s in (QKV, O, GATE_UP, DOWN)] == [1, 2, 1, 2]
    assert [splits(s, 1024) for s in (QKV, O, GATE_UP, DOWN)] == [1, 1, 1, 1]
    assert [splits(s, 2048) for s in (QKV, O, GATE_UP, DOWN, HEAD)] == [1, 1, 1, 1, 1]


def test_odd_sizes_never_split_what_tma_cannot_address():
    assert product(300, 100)._splits(4) == 1            # K not a multiple of 8: the plain kernel runs, unsplit
    assert product(300, 64)._splits(4) == 1             # a single K block cannot be split


def test_prompt_attention_orders_its_blocks_by_what_fits_the_l2_cache():
    # keys and values of the step's contexts: sequences x kv heads x tokens x 128 x 2 tensors x 2 bytes
    assert kernels.prefill_heads_first(1, 8, 128, 2048)
    assert kernels.prefill_heads_first(1, 8, 128, 16384)          # 67 MB
    assert not kernels.prefill_heads_first(1, 8, 128, 32768)      # 134 MB: one head after another
    assert not kernels.prefill_heads_first(8, 8, 128, 4096)       # eight such sequences: 134 MB
    assert kernels.prefill_heads_first(8, 8, 128, 32768, window=1024)   # a window bounds what a layer reads

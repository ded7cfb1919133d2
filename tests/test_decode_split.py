"""How decode attention's work is cut up (host-side policy; the SM count is given, no GPU)."""
import pytest

from rocml_b200 import kernels


@pytest.fixture(autouse=True)
def sms(monkeypatch):
    monkeypatch.setitem(kernels._sm_count, 0, 148)


@pytest.mark.parametrize("n_seqs", [1, 2, 8, 9, 64, 300])
@pytest.mark.parametrize("groups", [1, 8, 16])
@pytest.mark.parametrize("n_pages", [1, 2, 17, 20, 64])
def test_equal_split_covers_every_page_in_one_wave(n_seqs, groups, n_pages):
    blocks, ppb = kernels.decode_split(n_seqs, groups, n_pages)
    resident = 3 * 148
    if ppb == 0:
        # more (sequence, head group) pairs than run at once: one wave of blocks shares all pages
        assert n_pages >= 8 and resident < n_seqs * groups <= resident * 4 // 3 and 2 <= n_seqs <= 256
        assert 1 <= blocks and blocks * groups <= resident
        return
    assert ppb >= 1 and blocks >= 1
    assert blocks * ppb >= n_pages > (blocks - 1) * ppb          # every page, no empty block
    assert blocks == 1 or blocks * n_seqs * groups <= resident    # one wave, unless one block a sequence is already too many


def test_a_finer_split_is_cut_back_to_a_cluster_where_blocks_stay_short():
    assert kernels.decode_split(1, 8, 20) == (10, 2)      # 20 blocks would fit; 16 -> two pages a block -> ten blocks
    assert kernels.decode_split(1, 8, 64) == (16, 4)
    assert kernels.decode_split(8, 8, 20) == (5, 4)       # the wave allows six blocks a sequence
    assert kernels.decode_split(48, 8, 20) == (1, 20)
    assert kernels.decode_split(64, 8, 20) == (55, 0)     # 512 pairs do not run at once: 55 blocks a group share the pages
    assert kernels.decode_split(64, 8, 4) == (1, 4)       # too short to be worth it
    assert kernels.decode_split(100, 8, 20) == (1, 20)    # nearly two full waves of whole sequences


@pytest.mark.parametrize("n_seqs,groups,n_pages", [(4, 8, 65), (4, 8, 496), (64, 8, 100), (256, 2, 80), (64, 8, 17)])
def test_long_contexts_in_a_batch_share_the_blocks(n_seqs, groups, n_pages):
    blocks, ppb = kernels.decode_split(n_seqs, groups, n_pages)
    assert ppb == 0                                       # pages per block 0: the pages are shared out on the device
    assert 1 <= blocks <= 1024
    assert blocks * groups <= 3 * 148


def test_one_long_sequence_and_very_many_sequences_keep_the_equal_split():
    assert kernels.decode_split(1, 8, 512) == (16, 32)    # never more blocks than a cluster holds
    assert kernels.decode_split(1, 8, 128) == (16, 8)
    assert kernels.decode_split(3, 8, 500) == (16, 32)    # up to three long sequences: a cluster each
    assert kernels.decode_split(300, 8, 100)[1] > 0

"""Host-side pieces of the KV path that need no GPU: run canonicalisation, batch and group packing."""
import struct

import pytest
import torch

from aboleth_b200.kv import copy as kvcopy


def test_block_pairs_merge_into_maximal_runs():
    runs = kvcopy.canonicalize_block_runs([4, 5, 6, 30, 31, 9], [20, 21, 22, 3, 4, 5])
    assert runs == [(4, 20, 3), (30, 3, 2), (9, 5, 1)]
    # source consecutive but destination not: no merge
    assert kvcopy.canonicalize_block_runs([1, 2, 3], [7, 9, 10]) == [(1, 7, 1), (2, 9, 2)]
    # a descending pair never merges, an empty transfer has no runs
    assert kvcopy.canonicalize_block_runs([5, 4], [1, 0]) == [(5, 1, 1), (4, 0, 1)]
    assert kvcopy.canonicalize_block_runs([], []) == []
    with pytest.raises(ValueError):
        kvcopy.canonicalize_block_runs([1, 2], [1])
    # every page is covered exactly once, in order
    src, dst = [8, 9, 2, 3, 4, 11], [0, 1, 2, 3, 4, 5]
    covered = [(s + i, d + i) for s, d, n in kvcopy.canonicalize_block_runs(src, dst) for i in range(n)]
    assert covered == list(zip(src, dst))


def test_batches_pack_as_four_little_endian_words():
    packed = kvcopy.pack_batches([(0x1000, 0x2000, 4096, 0x3000), (0x1100, 0x2100, 512, 0x3008)], "cpu")
    assert packed.dtype == torch.uint8 and packed.numel() == 64
    words = struct.unpack("<8Q", bytes(packed.tolist()))
    assert words == (0x1000, 0x2000, 4096, 0x3000, 0x1100, 0x2100, 512, 0x3008)


def test_batches_that_publish_one_cell_share_one_arrival_counter():
    """Three batches name cell A, one names cell B: two groups, and a group's target is the worker
    total of all its batches, so cell A is published by the last worker of its last batch."""
    cell_a, cell_b = 0x5000, 0x5008
    group_of, target, groups = kvcopy.pack_groups([cell_a, cell_b, cell_a, cell_a], workers=16, device="cpu")
    assert groups == 2
    assert group_of.tolist() == [0, 1, 0, 0] and target.tolist() == [48, 16]
    assert group_of.dtype == target.dtype == torch.int32
    # one cell per batch degenerates to the per-batch count
    group_of, target, groups = kvcopy.pack_groups([1, 2, 3], workers=4, device="cpu")
    assert groups == 3 and group_of.tolist() == [0, 1, 2] and target.tolist() == [4, 4, 4]

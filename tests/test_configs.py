"""Synthetic workload generators: sizes, determinism and the properties the configurations ask for."""
import torch

from applied_ai_b200 import configs as C


def test_c1_shapes_and_determinism():
    x, w, m = C.c1_small()
    x2, w2, m2 = C.c1_small()
    assert x.shape == (512, 256) and w.shape == (4, 512, 256) and int(m.sum()) == 512
    assert torch.equal(x, x2) and torch.equal(w, w2) and torch.equal(m, m2)


def test_c2_group_sizes_are_multiples_of_128():
    m = C.m_sizes_blocks(8, 16384, 128, 1001)
    assert int(m.sum()) == 16384 and bool((m % 128 == 0).all()) and m.dtype == torch.int32


def test_c5_has_empty_and_unaligned_groups():
    m = C.m_sizes_zipf()
    assert int(m.sum()) == 8192 and m.numel() == 128
    assert int((m == 0).sum()) >= 8
    assert int(((m % 128) != 0).sum()) > 64
    assert int(m.max()) > 10 * int(m[m > 0].float().median())


def test_routing_topk():
    w, ids = C.routing(64, 8, 2, 3)
    assert ids.shape == (64, 2) and ids.dtype == torch.int32 and bool((ids[:, 0] != ids[:, 1]).all())
    assert bool((w[:, 0] >= w[:, 1]).all())

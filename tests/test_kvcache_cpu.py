"""Layout, sharing and the disk format of the whole-model INT8 KV cache container (no GPU)."""
import struct

import numpy as np
import pytest
import torch

from logos_b200.kvcache import KVCache, MAGIC


def _random_cache(seed=5, lens=(7, 3)):
    c = KVCache(3, 2, 4, 12, 16, device="cpu")
    g = torch.Generator().manual_seed(seed)
    c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=g, dtype=torch.int8))
    c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=g, dtype=torch.int8))
    c.ks.copy_(torch.rand(c.ks.shape, generator=g) + 0.01)
    c.vs.copy_(torch.rand(c.vs.shape, generator=g) + 0.01)
    c.set_lens(list(lens))
    return c


def test_layer_views_are_the_kernel_layout():
    c = KVCache(3, 2, 4, 12, 16, device="cpu")
    k, v, ks, vs = c.layer(1)
    assert k.shape == (2, 4, 12, 16) and k.is_contiguous() and v.is_contiguous()
    assert ks.shape == (2, 4) and ks.is_contiguous()
    assert k.data_ptr() == c.k.data_ptr() + 1 * 2 * 4 * 12 * 16       # a view of the arena, not a copy
    assert k.data_ptr() % 16 == 0
    assert c.nbytes() == 2 * 3 * 2 * 4 * 12 * 16 + 2 * 4 * 3 * 2 * 4 + 4 * 2


def test_bad_extents_are_rejected():
    with pytest.raises(ValueError):
        KVCache(0, 1, 1, 1, 16, device="cpu")
    with pytest.raises(ValueError):
        KVCache(1, 1, 1, 1, 24, device="cpu")       # rows must be whole 16-byte vectors


def test_dump_load_round_trip(tmp_path):
    c = _random_cache()
    path = str(tmp_path / "cache.bin")
    c.dump(path)
    raw = open(path, "rb").read()
    assert raw[:8] == MAGIC
    L_, B, H, S_max, DH, s_used, _, _ = struct.unpack("<8q", raw[8:72])
    assert (L_, B, H, S_max, DH, s_used) == (3, 2, 4, 12, 16, 7)
    assert len(raw) == 72 + 4 * 2 + 2 * 4 * 24 + 2 * 24 * 7 * 16    # only the rows in use travel
    d = KVCache.load(path, device="cpu")
    assert d.shape == c.shape
    assert torch.equal(d.lens, c.lens) and torch.equal(d.ks, c.ks) and torch.equal(d.vs, c.vs)
    assert torch.equal(d.k[:, :, :, :7], c.k[:, :, :, :7]) and torch.equal(d.v[:, :, :, :7], c.v[:, :, :, :7])
    assert int(d.k[:, :, :, 7:].abs().sum()) == 0                   # rows beyond the longest sequence start empty
    e = KVCache.load(path, device="cpu", s_max=32)                  # into a cache with more room
    assert e.shape == (3, 2, 4, 32, 16) and torch.equal(e.k[:, :, :, :7], c.k[:, :, :, :7])
    with pytest.raises(ValueError):
        KVCache.load(path, device="cpu", s_max=4)


def test_load_rejects_foreign_and_truncated_files(tmp_path):
    p = tmp_path / "x.bin"
    p.write_bytes(b"NOTACACHE" + bytes(100))
    with pytest.raises(ValueError):
        KVCache.load(str(p), device="cpu")
    c = _random_cache()
    q = tmp_path / "y.bin"
    c.dump(str(q))
    q.write_bytes(q.read_bytes()[:-10])
    with pytest.raises(ValueError):
        KVCache.load(str(q), device="cpu")


def test_share_prompt_copies_rows_scales_and_length():
    c = _random_cache(lens=(7, 0))
    c.share_prompt(0, [1])
    assert int(c.lens[1]) == 7
    assert torch.equal(c.k[:, 1, :, :7], c.k[:, 0, :, :7]) and torch.equal(c.v[:, 1, :, :7], c.v[:, 0, :, :7])
    assert torch.equal(c.ks[:, 1], c.ks[:, 0]) and torch.equal(c.vs[:, 1], c.vs[:, 0])

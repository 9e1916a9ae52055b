import torch

from mesh_b200.ops.philox import dropout, logical_index, philox4x32, uniform


def test_known_answers():
    # Random123 known-answer vectors for philox4x32 with 10 rounds
    kat = [((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
           ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
           ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
            (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1))]
    for ctr, key, want in kat:
        got = philox4x32(ctr, key)
        assert tuple(int(g) for g in got) == want


def test_uniform_statistics_and_independence_of_sites():
    e = torch.arange(1 << 16)
    u = uniform(e, seed=1234, execution=3, site=7)
    assert 0 <= float(u.min()) and float(u.max()) < 1 and abs(float(u.mean()) - 0.5) < 5e-3
    v = uniform(e, seed=1234, execution=3, site=8)
    assert abs(float(((u - 0.5) * (v - 0.5)).mean())) < 2e-3
    assert torch.equal(u, uniform(e, seed=1234, execution=3, site=7))


def test_dropout_mask_is_the_same_for_any_sharding():
    torch.manual_seed(0)
    x = torch.randn(4, 12, 6)
    full = dropout(x, 0.3, seed=99, execution=1, site=2)
    # contiguous shard of dim 1, and a striped shard of dim 1
    part = dropout(x[:, 4:8], 0.3, 99, 1, 2, full_shape=x.shape, slices=(None, slice(4, 8), None))
    assert torch.equal(part, full[:, 4:8])
    stripe = torch.arange(1, 12, 3)
    part = dropout(x[:, stripe], 0.3, 99, 1, 2, full_shape=x.shape, slices=(None, stripe, None))
    assert torch.equal(part, full[:, stripe])
    kept = (full != 0).float().mean()
    assert abs(float(kept) - 0.7) < 0.08
    assert torch.equal(logical_index((2, 3)), torch.arange(6).view(2, 3))

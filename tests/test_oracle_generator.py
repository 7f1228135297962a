"""CPU: the seeded generator, 16-bit conversions and the product's host fills against the oracle."""
import ml_dtypes
import numpy as np
import pytest


# Known-answer vectors of Philox4x32-10 from the Random123 distribution (kat_vectors):
# counter words, key words, expected output words.
PHILOX_KAT = [
    ([0, 0, 0, 0], [0, 0], [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
    ([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
    ([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0],
     [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]),
]


@pytest.mark.parametrize("ctr,key,want", PHILOX_KAT)
def test_philox_known_answers(oracle, ctr, key, want):
    assert oracle.philox4x32_10(ctr, key).tolist() == want


def test_fill_depends_only_on_seed_tensor_and_index(oracle):
    full = oracle.fill_normal((1000,), 7, 3, 1.0, 2.0)
    for off, n in ((0, 10), (1, 17), (2, 5), (3, 400), (513, 487)):
        assert np.array_equal(oracle.fill_normal((n,), 7, 3, 1.0, 2.0, elem_offset=off), full[off:off + n])
    assert not np.array_equal(oracle.fill_normal((1000,), 8, 3, 1.0, 2.0), full)
    assert not np.array_equal(oracle.fill_normal((1000,), 7, 4, 1.0, 2.0), full)
    u = oracle.fill_uniform((100000,), 2, 0, -1.0, 1.0)
    assert -1.0 < u.min() and u.max() < 1.0 and abs(u.mean()) < 0.01
    z = oracle.fill_normal((200000,), 0, 0, 0.0, 2.0)
    assert abs(z.mean()) < 0.02 and abs(z.std() - 2.0) < 0.02


def test_product_fills_match_oracle_bit_for_bit(oracle, ko):
    for off in (0, 5):
        assert np.array_equal(ko.fill_normal((333, 130), 0, 3, 0.0, 2.0, elem_offset=off),
                              oracle.fill_normal((333, 130), 0, 3, 0.0, 2.0, elem_offset=off))
        assert np.array_equal(ko.fill_uniform((333, 130), 9, 1, -1.0, 1.0, elem_offset=off),
                              oracle.fill_uniform((333, 130), 9, 1, -1.0, 1.0, elem_offset=off))
    # large enough to take the multi-threaded path of the product fill
    assert np.array_equal(ko.fill_normal((1 << 20,), 4, 0), oracle.fill_normal((1 << 20,), 4, 0))
    assert np.array_equal(ko.fill_uniform((500, 64), 3, 1, dtype=2), oracle.to_bf16_bits(oracle.fill_uniform((500, 64), 3, 1)))
    assert np.array_equal(ko.fill_normal((500, 64), 3, 1, dtype=1), oracle.to_f16_bits(oracle.fill_normal((500, 64), 3, 1)))


def test_causal_mask(oracle, ko):
    a = oracle.fill_normal((1100, 512), 4, 0, 0.0, 2.0)
    b = a.copy()
    oracle.causal_mask_(a, row_offset=700, block=512, value=-1e4)
    ko.fill_causal_mask_(b, row_offset=700, block=512, value=-1e4)
    assert np.array_equal(a, b)
    r = np.arange(1100)[:, None]
    c = np.arange(512)[None, :]
    masked = c > ((r + 700) % 512)
    assert np.all(a[masked] == np.float32(-1e4)) and np.all(a[~masked] != np.float32(-1e4))


def test_half_and_bfloat_rounding_matches_numpy(oracle):
    vals = np.concatenate([
        oracle.fill_normal((100000,), 5, 0, 0, 1), oracle.fill_normal((100000,), 5, 1, 0, 1e-6),
        oracle.fill_normal((100000,), 5, 2, 0, 3e4),
        np.array([65504, 65519.9, 65520, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 3e-8, 0, -0.0, np.inf, -np.inf], dtype=np.float32),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.to_f16_bits(vals), vals.astype(np.float16).view(np.uint16))
    assert np.array_equal(oracle.to_bf16_bits(vals), vals.astype(ml_dtypes.bfloat16).view(np.uint16))
    bits = np.arange(65536, dtype=np.uint16)
    for got, want in ((oracle.from_f16_bits(bits), bits.view(np.float16).astype(np.float32)),
                      (oracle.from_bf16_bits(bits), bits.view(ml_dtypes.bfloat16).astype(np.float32))):
        assert np.all((got == want) | (np.isnan(got) & np.isnan(want)))

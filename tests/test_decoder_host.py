"""Host-side guards of the decode engine that need no GPU: the KV cache is indexed on the device by
`positions`, so the host refuses to step past the cache before it launches anything."""

import pytest

from nf4_b200.decoder import NF4Decoder


def _shell(S, next_pos=0):
    dec = NF4Decoder.__new__(NF4Decoder)      # no device: only the fields the guard reads
    dec.S, dec.next_pos = S, next_pos
    return dec


def test_step_past_the_cache_is_refused_on_the_host():
    dec = _shell(S=4)
    for _ in range(4):
        dec._guard()
    assert dec.next_pos == 4
    with pytest.raises(RuntimeError, match="KV cache holds 4 positions"):
        dec._guard()
    assert dec.next_pos == 4                  # a refused step does not count


def test_set_positions_rejects_rows_outside_the_cache():
    dec = _shell(S=8)
    for bad in (-1, 8, 1000):
        with pytest.raises(ValueError, match="outside the cache"):
            dec.set_positions(bad)

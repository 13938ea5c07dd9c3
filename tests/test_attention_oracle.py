"""The attention oracle: tile-program form against the textbook form (no GPU)."""

import pytest
import torch

import cases
from oracle import attention_oracle


@pytest.mark.parametrize("seq,causal", [(128, True), (256, True), (200, True), (256, False), (96, False)])
def test_tiles_match_plain(seq, causal):
    q, k, v = (cases.gen((2 * seq, 128), "normal", s).reshape(2, seq, 128) for s in (0, 1, 2))
    a = attention_oracle.attention_tiles(q, k, v, causal, 128 ** -0.5)
    b = attention_oracle.attention_plain(q, k, v, causal, 128 ** -0.5)
    assert (a.float() - b.float()).abs().max() <= 2 ** -7 * b.float().abs().max()


def test_causal_first_row_is_first_value():
    q, k, v = (cases.gen((256, 128), "normal", s).reshape(1, 256, 128) for s in (3, 4, 5))
    o = attention_oracle.attention_tiles(q, k, v, True, 128 ** -0.5)
    assert torch.equal(o[0, 0], v[0, 0])

"""The plain implementation against the reference's shipped fixture
(tests/fixtures/dense of d9beuD/rust-mlx: a 2-layer float32 Qwen3 made by its
oracle script, scripts/dense_oracle.py).  The oracle ran on an Apple GPU, whose
matrix products are not exact in 32-bit, hence 5e-3 on logits whose range is
about -1.4 .. 1.7; the 32 greedy tokens must be equal.  A copy of what the plain
implementation gives for this fixture lies in tests/golden/ and is compared
bit-tight, so the test still says something where the reference is not mounted."""
import json
import os

import pytest
import torch

import plain_qwen3 as plain

# the reference's checkout, beside this repository unless REFERENCE_DIR says otherwise
REFERENCE = os.environ.get("REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "..", "reference"))
FIXTURE = os.path.join(REFERENCE, "tests", "fixtures", "dense")
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "dense_fixture_plain.json")


@pytest.mark.skipif(not os.path.isdir(FIXTURE), reason="reference fixture not mounted")
def test_plain_matches_reference_oracle():
    oracle = json.load(open(os.path.join(FIXTURE, "oracle.json")))
    m = plain.PlainModel(FIXTURE)
    logits = m.logits(oracle["prompt"])[-1]
    want = torch.tensor(oracle["prefill_logits"], dtype=torch.float64)
    assert (logits - want).abs().max().item() < 5e-3
    assert m.greedy(oracle["prompt"], len(oracle["tokens"])) == oracle["tokens"]


@pytest.mark.skipif(not os.path.isdir(FIXTURE), reason="reference fixture not mounted")
def test_plain_matches_its_committed_output():
    gold = json.load(open(GOLDEN))
    m = plain.PlainModel(FIXTURE)
    logits = m.logits(gold["prompt"])[-1]
    assert (logits - torch.tensor(gold["last_logits"], dtype=torch.float64)).abs().max().item() < 1e-9
    assert m.greedy(gold["prompt"], len(gold["tokens"])) == gold["tokens"]


def test_wrong_rotation_pairing_is_far_from_oracle():
    """Interleaved pairs (2j, 2j+1) instead of (j, j+half) must not pass: guards the
    convention of kernels/text_rope.metal:3-14."""
    if not os.path.isdir(FIXTURE):
        pytest.skip("reference fixture not mounted")
    oracle = json.load(open(os.path.join(FIXTURE, "oracle.json")))
    m = plain.PlainModel(FIXTURE)
    good = plain.rope

    def interleaved(x, positions, theta, rotary_dim, inv_freq=None):
        half = rotary_dim // 2
        perm = torch.cat([torch.arange(0, rotary_dim, 2), torch.arange(1, rotary_dim, 2)])
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(rotary_dim)
        return good(x[..., perm], positions, theta, rotary_dim, inv_freq)[..., inv]

    plain.rope = interleaved
    try:
        logits = m.logits(oracle["prompt"])[-1]
    finally:
        plain.rope = good
    want = torch.tensor(oracle["prefill_logits"], dtype=torch.float64)
    assert (logits - want).abs().max().item() > 0.1

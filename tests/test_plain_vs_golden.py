"""The plain implementation against arrays the reference's own model code produced
(tests/golden/make_golden.py), and against itself in float64."""

import tempfile
from pathlib import Path

import numpy as np
import pytest

import dli_b200
from tests.plain import llama_plain as plain
from tests.tiny_configs import TINY

GOLDEN = Path(__file__).parent / "golden"


@pytest.fixture(scope="module", params=sorted(TINY))
def case(request):
    cfg, seed, _ = TINY[request.param]
    with tempfile.TemporaryDirectory() as tmp:
        dli_b200.write_model_dir(tmp, cfg, seed)
        weights = plain.read_safetensors(Path(tmp) / "model.safetensors")
    gold = np.load(GOLDEN / f"{request.param}.npz")
    checksum = sum(float(np.abs(w.astype(np.float64)).sum()) for w in weights.values())
    assert abs(checksum - float(gold["weight_checksum"])) < 1e-6 * checksum, "random weights differ from the golden run's"
    return cfg, weights, gold


def test_logits_match_reference(case):
    cfg, weights, gold = case
    logits = plain.forward(cfg, weights, gold["token_ids"])
    np.testing.assert_allclose(logits[gold["positions"]], gold["logits"], atol=1e-4, rtol=0)


def test_inverse_frequencies_match_reference(case):
    cfg, _, gold = case
    inv = plain.inverse_frequencies(plain.read_config(cfg))
    np.testing.assert_allclose(inv, gold["inv_freq"], rtol=3e-7, atol=0)


def test_greedy_matches_reference(case):
    cfg, weights, gold = case
    assert plain.greedy_generate(cfg, weights, gold["token_ids"][:9].tolist(), 16) == gold["greedy"].tolist()


def test_float64_agrees(case):
    cfg, weights, gold = case
    ids = gold["token_ids"][:24]
    a = plain.forward(cfg, weights, ids)
    b = plain.forward(cfg, weights, ids, dtype=np.float64)
    np.testing.assert_allclose(a, b, atol=2e-5, rtol=0)


def test_llama3_bands():
    """All three frequency bands appear in tiny_b: kept, interpolated, divided by the factor."""
    from tests.tiny_configs import TINY_B

    c = plain.read_config(TINY_B)
    scaled = plain.inverse_frequencies(c)
    base = plain.inverse_frequencies({**c, "rope_type": "default"})
    ratio = scaled / base
    assert np.allclose(ratio[:2], 1.0) and np.allclose(ratio[3:], 1 / 8, rtol=1e-6)
    assert 1 / 8 < ratio[2] < 1.0


def test_sampling_distribution_matches_reference():
    """The probabilities the reference's sampler draws from (tests/golden/make_sampling_golden.py), row by
    row, against the plain sampler's; and its greedy choices, ties included."""
    data = np.load(GOLDEN / "sampling_probs.npz")
    logits, settings = data["logits"], data["settings"]
    for i, want in zip(data["rows"], data["probs"]):
        t, k, p = settings[i % len(settings)]
        got = plain.filtered_probabilities(logits[i], float(t), int(k), float(p))
        assert (got > 0).tolist() == (want > 0).tolist(), f"row {i}: another set of tokens survives"
        np.testing.assert_allclose(got, want, atol=2e-6, err_msg=f"row {i}")
    for i, token in data["greedy"]:
        t, k, p = settings[i % len(settings)]
        assert plain.sample_token(logits[i], float(t), int(k), float(p), seed=1, draw=0) == token

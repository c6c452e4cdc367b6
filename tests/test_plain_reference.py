"""The plain implementation against the reference's own modules (stored logits) and against itself."""

import hashlib
import json
from pathlib import Path

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.tiny_configs import TINY, TINY_C, tiny_weights

GOLDEN = Path(__file__).parent / "golden"


def _checksum(weights):
    h = hashlib.sha256()
    for name in sorted(weights):
        h.update(name.encode())
        h.update(weights[name].to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("tag", ["a", "b"])
def test_plain_matches_reference_modules(tag):
    record = json.loads((GOLDEN / f"qwen3_tiny_{tag}.json").read_text())
    cfg = record["config"]
    assert cfg == TINY[tag], "the stored logits were made for another configuration"
    weights = tiny_weights(cfg, seed=record["seed"])
    # the tests' generator is plain integer hashing: the weights are the same everywhere, so a
    # mismatch means the generator or the stored file was changed without the other
    assert _checksum(weights) == record["weights_sha256"], "the stored logits were made with other weights"
    for ids, want in zip(record["sequences"], record["logits"]):
        want = torch.tensor(want, dtype=torch.float64)
        got32 = plain.forward_logits(weights, cfg, ids, dtype=torch.float32).double()
        got64 = plain.forward_logits(weights, cfg, ids, dtype=torch.float64)
        scale = want.abs().max()
        assert (got32 - want).abs().max() <= 2e-5 * scale
        assert (got64 - want).abs().max() <= 2e-5 * scale


def test_rope_is_a_rotation_and_position_zero_is_identity():
    x = torch.randn(5, 3, 16, dtype=torch.float64)
    ang = plain.rope_angles([0, 1, 2, 3, 100], 16, 1e4)
    y = plain.apply_rope(x, ang)
    assert torch.allclose(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # q.k after rotation depends on the distance only
    q = torch.randn(1, 1, 16, dtype=torch.float64)
    k = torch.randn(1, 1, 16, dtype=torch.float64)
    a = (plain.apply_rope(q, plain.rope_angles([7], 16, 1e4)) * plain.apply_rope(k, plain.rope_angles([3], 16, 1e4))).sum()
    b = (plain.apply_rope(q, plain.rope_angles([24], 16, 1e4)) * plain.apply_rope(k, plain.rope_angles([20], 16, 1e4))).sum()
    assert abs(a - b) < 1e-5


def test_attention_causal_and_window():
    T, nq, nkv, d = 12, 4, 2, 8
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nq, nkv, nkv))
    full = plain.causal_attention(q, k, v, scale=d**-0.5)
    # the first query sees only the first key
    assert torch.allclose(full[0, 0], v[0, 0])
    # changing a later key does not change earlier outputs
    k2 = k.clone(); k2[7] += 1.0
    assert torch.allclose(plain.causal_attention(q, k2, v, scale=d**-0.5)[:7], full[:7])
    # a window of T or more is no window; a window of 1 returns the own value
    assert torch.allclose(plain.causal_attention(q, k, v, scale=d**-0.5, window=T), full)
    w1 = plain.causal_attention(q, k, v, scale=d**-0.5, window=1)
    assert torch.allclose(w1[:, 0], v[:, 0]) and torch.allclose(w1[:, 3], v[:, 1])
    # window 3: output at t equals full attention over keys t-2..t alone
    w3 = plain.causal_attention(q, k, v, scale=d**-0.5, window=3)
    t = 9
    ref = plain.causal_attention(q[t - 2 : t + 1], k[t - 2 : t + 1], v[t - 2 : t + 1], scale=d**-0.5)[-1]
    assert torch.allclose(w3[t], ref)


def test_prefix_logits_do_not_depend_on_what_follows():
    cfg = TINY_C
    w = tiny_weights(cfg, seed=5, sharp=3.0)
    ids = torch.randint(0, cfg["vocab_size"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward_logits(w, cfg, ids)
    part = plain.forward_logits(w, cfg, ids[:29])
    assert torch.allclose(whole[:29], part, atol=1e-10)
    assert plain.layer_windows(cfg) == [None, 24, 24, None]


def test_sampler_greedy_and_seeded():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert plain.sample_token(logits, 0.0, key=1) == 1
    draws = [plain.sample_token(logits, 1.0, key=k) for k in range(200)]
    assert draws == [plain.sample_token(logits, 1.0, key=k) for k in range(200)]
    counts = [draws.count(i) for i in range(4)]
    assert counts[1] > counts[0] and counts[2] > counts[3] and counts[1] + counts[2] > 120


# -- the attention core against the reference's own attention path (flash-attn on a GPU) ----------
#
# tests/golden/make_golden_flash.py stored what the reference's FlashSDPA returns for bfloat16
# q, k, v, and the logits of its unmodified Transformer in bfloat16.  flash-attn rounds the
# probabilities to bfloat16 before the second product and returns bfloat16: 2^-9 per rounding on
# values of the outputs' size, so 2e-2 of the largest output is a wide bound for the core alone;
# the whole model in bfloat16 (every activation rounded, several layers) gets the engine's own
# bfloat16 bound of 4e-2.  A wrong head mapping moves both by more than the largest value.

FLASH_TOLERANCE = 2e-2
FLASH_MODEL_TOLERANCE = 4e-2


def _wrong_head_mapping(q, k, v, *, scale, window=None):
    """Query head g reads KV head g % nkv instead of g // group: wrong whenever 1 < nkv < nq."""
    nq, nkv = q.shape[1], k.shape[1]
    pick = [g % nkv for g in range(nq)]
    return _right_attention(q, k[:, pick], v[:, pick], scale=scale, window=window)


_right_attention = plain.causal_attention


def _flash_inputs(shape):
    from tests.golden.make_golden_flash import attention_inputs

    return tuple(t.double() for t in attention_inputs(tuple(shape)))


def test_attention_core_matches_the_references_flash_attention():
    record = json.loads((GOLDEN / "flash_attention.json").read_text())
    assert len(record["cases"]) >= 5
    caught = 0
    for case in record["cases"]:
        T, nq, nkv, d = case["shape"]
        q, k, v = _flash_inputs(case["shape"])
        want = torch.tensor(case["out"], dtype=torch.float64).view(T, nq, d)
        got = plain.causal_attention(q, k, v, scale=d**-0.5)
        scale = want.abs().max()
        assert (got - want).abs().max() <= FLASH_TOLERANCE * scale, f"shape {case['shape']}"
        if 1 < nkv < nq:
            bad = _wrong_head_mapping(q, k, v, scale=d**-0.5)
            assert (bad - want).abs().max() > 10 * FLASH_TOLERANCE * scale, "the check cannot tell a wrong head mapping"
            caught += 1
        # the scale is head_dim^-0.5: another one is told apart as well
        other = plain.causal_attention(q, k, v, scale=1.0 / d)
        if T > 4:
            assert (other - want).abs().max() > 2 * FLASH_TOLERANCE * scale, "the check cannot tell a wrong scale"
    assert caught >= 2


@pytest.mark.parametrize("tag", ["a", "b"])
def test_plain_matches_the_references_model_with_flash_attention(tag, monkeypatch):
    from tests.golden.make_golden_flash import rounded_weights, weights_checksum

    record = json.loads((GOLDEN / f"qwen3_flash_{tag}.json").read_text())
    cfg = record["config"]
    assert cfg == TINY[tag], "the stored logits were made for another configuration"
    weights = rounded_weights(cfg)
    assert weights_checksum(weights) == record["weights_sha256"], "the stored logits were made with other weights"
    weights = {k: v.float() for k, v in weights.items()}
    worst_right, worst_wrong = 0.0, 0.0
    for ids, want in zip(record["sequences"], record["logits"]):
        want = torch.tensor(want, dtype=torch.float64)
        got = plain.forward_logits(weights, cfg, ids, dtype=torch.float64)
        scale = want.abs().max()
        worst_right = max(worst_right, float((got - want).abs().max() / scale))
        if len(ids) > 8:
            monkeypatch.setattr(plain, "causal_attention", _wrong_head_mapping)
            bad = plain.forward_logits(weights, cfg, ids, dtype=torch.float64)
            monkeypatch.setattr(plain, "causal_attention", _right_attention)
            worst_wrong = max(worst_wrong, float((bad - want).abs().max() / scale))
    assert worst_right <= FLASH_MODEL_TOLERANCE, f"plain model strays {worst_right:.3g} from the reference's bfloat16 logits"
    assert worst_wrong > 5 * FLASH_MODEL_TOLERANCE, "the comparison cannot tell a wrong head mapping"

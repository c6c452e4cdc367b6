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
    if _checksum(weights) != record["weights_sha256"]:
        pytest.skip("this torch draws other random weights than the one the stored logits were made with")
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

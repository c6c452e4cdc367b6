"""Each kernel alone against a plain reference, at sizes other than the engine tests use."""

import math

import numpy as np
import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


TOL = {torch.float32: 2e-6, torch.bfloat16: 1e-2}


# ---------------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,H,T", [(37, 50, 9), (1000, 1032, 3)])
def test_embed_gather(dtype, V, H, T):
    from tokensprint_b200 import ops

    table = torch.randn(V, H, device=DEV).to(dtype)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    hidden = torch.empty(T, H, device=DEV)
    ops.embed_gather(hidden, table, ids)
    assert torch.equal(hidden.cpu(), plain.embedding(table.float().cpu(), ids.tolist()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,eps", [(5, 96, 1e-5), (3, 1000, 1e-6), (2, 4104, 1e-3), (1, 7, 1e-6)])
def test_add_rmsnorm(dtype, T, H, eps):
    from tokensprint_b200 import ops

    hidden = torch.randn(T, H, device=DEV) * 3
    delta = torch.randn(T, H, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(H, device=DEV)
    out = torch.empty(T, H, device=DEV, dtype=dtype)
    h0 = hidden.clone()
    ops.add_rmsnorm(hidden, delta, w, out, eps)
    want_h = h0.double() + delta.double()
    assert rel_err(hidden, want_h) < 2e-7
    assert rel_err(out, plain.rms_norm(want_h.cpu(), w.double().cpu(), eps)) < TOL[dtype]
    # without a delta the residual is untouched; with row_index only those rows are read
    h1 = hidden.clone()
    ops.add_rmsnorm(hidden, None, w, out, eps)
    assert torch.equal(hidden, h1)
    rows = torch.tensor([T - 1, 0], device=DEV, dtype=torch.int32)
    out2 = torch.empty(2, H, device=DEV, dtype=dtype)
    ops.add_rmsnorm(hidden, delta, w, out2, eps, rows)
    assert torch.equal(hidden, h1)
    want = plain.rms_norm((h1.double() + delta.double()).cpu()[[T - 1, 0]], w.double().cpu(), eps)
    assert rel_err(out2, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    from tokensprint_b200 import ops

    T, I = 7, 136
    gu = (torch.randn(T, 2 * I, device=DEV) * 4).to(dtype)
    out = torch.empty(T, I, device=DEV, dtype=dtype)
    ops.swiglu(gu, out)
    g, u = gu[:, :I].double().cpu(), gu[:, I:].double().cpu()
    assert rel_err(out, g * torch.sigmoid(g) * u) < TOL[dtype]


@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (70, 130, 100), (257, 64, 1025)])
def test_sgemm_is_true_float32(M, N, K):
    from tokensprint_b200 import ops

    a = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    out = torch.empty(M, N, device=DEV)
    ops.sgemm_nt(a, w, out)
    want = a.double() @ w.double().T
    # float32 products summed in float32: error grows like sqrt(K) * 2^-24, far below any
    # reduced-precision matrix mode (2^-11 per product)
    assert float((out.double() - want).abs().max()) < 4e-7 * math.sqrt(K) * float(want.abs().max())
    # a row's result does not depend on the rows beside it
    out1 = torch.empty(1, N, device=DEV)
    ops.sgemm_nt(a[M - 1 :], w, out1)
    assert torch.equal(out1[0], out[M - 1])


# ---------------------------------------------------------------------------
# q/k norm + rope + store


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [11, 64, 130, 300])
@pytest.mark.parametrize("nq,nkv,d,theta,rot", [(5, 1, 48, 5e4, 48), (4, 2, 16, 1e4, 16), (3, 3, 80, 1e6, 32), (8, 2, 256, 1e6, 256), (32, 8, 128, 1e6, 128)])
def test_qk_norm_rope_store(dtype, nq, nkv, d, theta, rot, T):
    from tokensprint_b200 import ops

    page = 4
    pages = -(-T // page) + 6
    eps = 1e-5
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV).to(dtype)
    positions = torch.randint(0, 3000, (T,), device=DEV, dtype=torch.int32)
    positions[:11] = torch.tensor([0, 1, 2, 3, 500, 501, 40000, 7, 8, 9, 10], device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * page, device=DEV)[:T].to(torch.int32)
    slots[5] = -1  # not stored
    qw = 1 + 0.2 * torch.randn(d, device=DEV)
    kw = 1 + 0.2 * torch.randn(d, device=DEV)
    inv_freq = plain.rope_inverse_frequencies(rot, theta).to(DEV)
    q_out = torch.empty(T, nq * d, device=DEV, dtype=dtype)
    kc = torch.full((pages, page, nkv, d), 7.0, device=DEV, dtype=dtype)
    vc = torch.full((pages, page, nkv, d), 7.0, device=DEV, dtype=dtype)
    ops.qk_norm_rope_store(qkv, q_out, kc, vc, slots, positions, qw, kw, eps, inv_freq, nq, nkv, d)

    x = qkv.double().cpu()
    q = x[:, : nq * d].view(T, nq, d)
    k = x[:, nq * d : (nq + nkv) * d].view(T, nkv, d)
    v = x[:, (nq + nkv) * d :].view(T, nkv, d)
    ang = plain.rope_angles(positions.tolist(), rot, theta)

    def enc(t, w):
        t = plain.rms_norm(t, w.double().cpu(), eps)
        return torch.cat([plain.apply_rope(t[..., :rot], ang), t[..., rot:]], dim=-1)

    # float32 angles reach 4e4 rad: sin/cos of the device and of the host agree to ~1e-6 there
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    assert rel_err(q_out.view(T, nq, d), enc(q, qw)) < tol
    kc_flat, vc_flat = kc.view(-1, nkv, d), vc.view(-1, nkv, d)
    want_k = enc(k, kw)
    touched = set()
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        touched.add(s)
        assert rel_err(kc_flat[s], want_k[t]) < tol
        assert torch.equal(vc_flat[s].double().cpu(), v[t])
    for s in range(pages * page):
        if s not in touched:
            assert float(kc_flat[s].float().min()) == 7.0 and float(vc_flat[s].float().max()) == 7.0


# ---------------------------------------------------------------------------
# attention


def paged_case(seqs, nq, nkv, d, page, dtype, seed=0, shuffle=True, poison=True):
    """Random q for the new tokens of every sequence, random k/v for its whole context,
    scattered over shuffled pages.  seqs: list of (q_len, ctx_len).  Returns the tensors
    the kernels take and per-sequence dense (q, k, v)."""
    g = torch.Generator().manual_seed(seed)
    B = len(seqs)
    blocks = [-(-c // page) for _, c in seqs]
    total_pages = sum(blocks) + 3
    order = torch.randperm(total_pages, generator=g).tolist() if shuffle else list(range(total_pages))
    fill = float("nan") if poison else 0.0
    kc = torch.full((total_pages, page, nkv, d), fill, dtype=torch.float32)
    vc = torch.full((total_pages, page, nkv, d), fill, dtype=torch.float32)
    table = torch.full((B, max(blocks)), -1, dtype=torch.int32)
    qs, dense = [], []
    positions, seq_index, cu, ctxs = [], [], [0], []
    used = 0
    for b, (ql, ctx) in enumerate(seqs):
        q = torch.randn(ql, nq, d, generator=g)
        k = torch.randn(ctx, nkv, d, generator=g)
        v = torch.randn(ctx, nkv, d, generator=g)
        dense.append([q, k, v])
        qs.append(q)
        for i in range(blocks[b]):
            table[b, i] = order[used]
            used += 1
        positions += list(range(ctx - ql, ctx))
        seq_index += [b] * ql
        cu.append(cu[-1] + ql)
        ctxs.append(ctx)
    case = dict(B=B, nq=nq, nkv=nkv, d=d, page=page, dtype=dtype, seqs=seqs, dense=dense, table=table, kc=kc, vc=vc,
                positions=positions, seq_index=seq_index, cu=cu, ctxs=ctxs)
    return case


def finish_case(case):
    """Rounds to the dtype, scatters k/v into the pages and moves everything to the device."""
    dtype, page = case["dtype"], case["page"]
    for b, (q, k, v) in enumerate(case["dense"]):
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        case["dense"][b] = [q, k, v]
        for j in range(k.shape[0]):
            pg = int(case["table"][b, j // page])
            case["kc"][pg, j % page] = k[j]
            case["vc"][pg, j % page] = v[j]
    case["q"] = torch.cat([d[0] for d in case["dense"]]).reshape(-1, case["nq"] * case["d"]).to(DEV, dtype)
    for name in ("kc", "vc"):
        case[name] = case[name].to(DEV, dtype)
    case["table"] = case["table"].to(DEV)
    for name in ("positions", "seq_index", "cu", "ctxs"):
        case[name] = torch.tensor(case[name], dtype=torch.int32, device=DEV)
    return case


def plain_attention(case, window=0):
    outs = []
    for (ql, ctx), (q, k, v) in zip(case["seqs"], case["dense"]):
        qfull = torch.zeros(ctx, case["nq"], case["d"], dtype=torch.float64)
        qfull[ctx - ql :] = q.double()
        o = plain.causal_attention(qfull, k.double(), v.double(), scale=case["d"] ** -0.5, window=window or None)
        outs.append(o[ctx - ql :])
    return torch.cat(outs).reshape(-1, case["nq"] * case["d"])


def run_simple(case, window=0):
    from tokensprint_b200 import ops

    out = torch.full_like(case["q"], float("nan"))
    ops.attention_paged_simple(case["q"], case["kc"], case["vc"], out, case["positions"], case["seq_index"], case["table"],
                               case["page"], case["nq"], case["nkv"], case["d"], case["d"] ** -0.5, window)
    return out


def run_mma(case, window=0, splits=1, keys_per_split=0, fuse_merge=True):
    from tokensprint_b200 import ops

    out = torch.full_like(case["q"], float("nan"))
    T = case["q"].shape[0]
    scratch = None
    if splits > 1:
        scratch = torch.full((ops.attention_scratch_floats(T * case["nq"], splits, case["d"]),), float("nan"), device=DEV)
    max_q = max(ql for ql, _ in case["seqs"])
    ops.attention_paged_mma(case["q"], case["kc"], case["vc"], out, case["cu"], case["ctxs"], case["table"], case["seq_index"],
                            case["page"], case["B"], max_q, case["nq"], case["nkv"], case["d"], case["d"] ** -0.5, window, splits, scratch,
                            keys_per_split, fuse_merge)
    return out


MIXED = [(1, 1), (1, 77), (5, 5), (3, 130), (64, 64), (37, 200), (2, 65), (1, 64), (130, 131)]
DECODE = [(1, 1), (1, 63), (1, 64), (1, 65), (1, 300), (1, 1000), (1, 129)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(4, 2, 16, 16, 0), (5, 1, 48, 4, 0), (6, 3, 32, 32, 24), (2, 2, 80, 1, 7), (3, 1, 272, 8, 0)])
def test_attention_simple(dtype, nq, nkv, d, page, window):
    case = finish_case(paged_case(MIXED, nq, nkv, d, page, dtype, seed=d))
    got = run_simple(case, window)
    want = plain_attention(case, window)
    assert rel_err(got, want) < (3e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize(
    "nq,nkv,d,page,window",
    [(4, 2, 16, 16, 0), (5, 1, 48, 4, 0), (6, 3, 32, 32, 24), (2, 2, 80, 1, 7), (32, 8, 128, 16, 0), (8, 1, 64, 16, 100),
     (2, 1, 256, 8, 0), (20, 1, 112, 16, 0), (4, 4, 96, 256, 0)],
)
def test_attention_mma_mixed(nq, nkv, d, page, window):
    case = finish_case(paged_case(MIXED, nq, nkv, d, page, torch.bfloat16, seed=d + 1))
    got = run_mma(case, window)
    want = plain_attention(case, window)
    assert rel_err(got, want) < 1e-2


@pytest.mark.parametrize("splits", [1, 2, 5, 8, 32])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(32, 8, 128, 16, 0), (4, 2, 16, 16, 0), (16, 1, 64, 32, 0), (5, 1, 48, 4, 90), (40, 2, 80, 16, 0),
                                                  (8, 2, 128, 8, 200), (4, 1, 128, 256, 0), (6, 2, 192, 64, 0), (2, 1, 256, 16, 300), (8, 8, 64, 128, 0)])
def test_attention_mma_decode_with_key_splits(splits, nq, nkv, d, page, window):
    case = finish_case(paged_case(DECODE, nq, nkv, d, page, torch.bfloat16, seed=3 * d))
    got = run_mma(case, window, splits)
    want = plain_attention(case, window)
    assert rel_err(got, want) < 1e-2
    # the merge as a kernel of its own gives the same, and twice in a row (the tickets reset)
    assert rel_err(run_mma(case, window, splits, fuse_merge=False), want) < 1e-2
    assert torch.equal(run_mma(case, window, splits), got)
    # 2..8 splits merge inside a thread-block cluster by default; through scratch and a second kernel it is the same
    from tokensprint_b200 import ops

    lib = ops._build.load_variant("attention_mma", {"TS_HEAD_DIM": d})
    assert lib.ts_attention_mma_cluster_merge() == 1
    lib.ts_attention_mma_set_cluster_merge(0)
    try:
        assert rel_err(run_mma(case, window, splits), want) < 1e-2
    finally:
        lib.ts_attention_mma_set_cluster_merge(1)
    # keys and values come by the copy engine where head and page sizes allow it; by the threads' own copies it is the same
    lib.ts_attention_mma_set_decode_tma(0)
    try:
        assert rel_err(run_mma(case, window, splits), want) < 1e-2
    finally:
        lib.ts_attention_mma_set_decode_tma(1)
    torch.cuda.synchronize()
    ops.check_device_errors()


def run_flat(case, window=0, ctas=0):
    from tokensprint_b200 import ops

    out = torch.full_like(case["q"], float("nan"))
    max_q = max(ql for ql, _ in case["seqs"])
    ops.attention_decode_flat(case["q"], case["kc"], case["vc"], out, case["cu"], case["ctxs"], case["table"], case["seq_index"],
                              case["page"], case["B"], max_q, case["nq"], case["nkv"], case["d"], case["d"] ** -0.5, window, ctas)
    return out


@pytest.mark.parametrize("ctas", [0, 1, 2, 7, 23, 150])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(32, 8, 128, 16, 0), (16, 1, 64, 32, 0), (8, 2, 128, 8, 200), (4, 1, 128, 256, 0),
                                                  (6, 2, 192, 64, 0), (2, 1, 256, 16, 300), (8, 8, 64, 128, 0), (12, 3, 128, 16, 90)])
def test_attention_decode_flat(ctas, nq, nkv, d, page, window):
    """The even-share decode kernel: the key blocks of all (sequence, KV head) pairs are one list that
    `ctas` CTAs divide evenly.  One CTA walks every pair; a few walk several pairs each and share some;
    many take a block or two each (and some nothing)."""
    from tokensprint_b200 import ops

    case = finish_case(paged_case(DECODE, nq, nkv, d, page, torch.bfloat16, seed=7 * d + nq))
    want = plain_attention(case, window)
    got = run_flat(case, window, ctas)
    assert rel_err(got, want) < 1e-2
    assert torch.equal(run_flat(case, window, ctas), got)
    torch.cuda.synchronize()
    ops.check_device_errors()


@pytest.mark.parametrize("ctas", [0, 5])
def test_attention_decode_flat_rows_of_several_tokens_and_lanes_without_a_sequence(ctas):
    """Sequences that bring up to four tokens (16 rows with four heads per KV head), sequences of a
    fixed-size batch that bring none, and token lanes that belong to no sequence (their output is zero)."""
    from tokensprint_b200 import ops

    nq, nkv, d, page = 8, 2, 128, 16
    seqs = [(4, 4), (2, 65), (1, 64), (3, 500), (4, 129), (1, 1)]
    case = finish_case(paged_case(seqs, nq, nkv, d, page, torch.bfloat16, seed=11))
    want = plain_attention(case, 0)
    T = case["q"].shape[0]
    # two more sequences without tokens, three more token lanes without a sequence
    B = case["B"] + 2
    cu = torch.cat([case["cu"], case["cu"][-1:].repeat(2)])
    ctxs = torch.cat([case["ctxs"], torch.zeros(2, dtype=torch.int32, device=DEV)])
    table = torch.cat([case["table"], torch.full((2, case["table"].shape[1]), -1, dtype=torch.int32, device=DEV)])
    q = torch.cat([case["q"], torch.randn(3, nq * d, device=DEV).bfloat16()])
    seq_index = torch.cat([case["seq_index"], torch.full((3,), -1, dtype=torch.int32, device=DEV)])
    out = torch.full_like(q, float("nan"))
    ops.attention_decode_flat(q, case["kc"], case["vc"], out, cu, ctxs, table, seq_index, page, B, 4, nq, nkv, d, d ** -0.5, 0, ctas)
    assert rel_err(out[:T], want) < 1e-2
    assert float(out[T:].float().abs().max()) == 0.0
    torch.cuda.synchronize()
    ops.check_device_errors()


@pytest.mark.parametrize("ctas", [0, 3])
@pytest.mark.parametrize("target", ["first", "far", "page_edge_before", "page_edge_after", "block_edge", "last", "window_first", "window_out"])
def test_attention_decode_flat_finds_one_key_that_stands_out(target, ctas):
    nq, nkv, d, page, ctx = 4, 1, 64, 16, 700
    window = 0
    where = {"first": 0, "far": 3, "page_edge_before": 16 * 20 - 1, "page_edge_after": 16 * 20, "block_edge": 64 * 7,
             "last": ctx - 1}.get(target)
    if target == "window_first":
        window, where = 100, ctx - 100
    if target == "window_out":
        window, where = 100, ctx - 101
    case = paged_case([(1, 90), (1, ctx), (1, 200)], nq, nkv, d, page, torch.bfloat16, seed=5)
    q, k, v = case["dense"][1]
    k.mul_(0.05)
    k[where, 0] = q[0, 2] * 3.0  # head 2's query finds itself at `where`
    v[where, 0] = 10.0
    case = finish_case(case)
    got = run_flat(case, window, ctas)
    head2 = got.view(3, nq, d)[1, 2].float()
    if target == "window_out":
        assert float(head2.abs().max()) < 5.0, "a key outside the window was seen"
    else:
        assert float((head2 - 10.0).abs().max()) < 0.05, f"the key at {where} was not found"
    assert rel_err(got, plain_attention(case, window)) < 1e-2


def test_attention_decode_flat_long_and_short_sequences_together():
    """One sequence of 20,000 keys beside short ones: the long one is shared by nearly all CTAs,
    the short ones lie inside single CTAs."""
    from tokensprint_b200 import ops

    nq, nkv, d, page = 8, 2, 128, 16
    case = finish_case(paged_case([(1, 30), (1, 20000), (1, 70), (1, 3000), (1, 64)], nq, nkv, d, page, torch.bfloat16, seed=13))
    assert rel_err(run_flat(case, 0, 0), plain_attention(case, 0)) < 1e-2
    torch.cuda.synchronize()
    ops.check_device_errors()


def test_attention_decode_flat_says_what_it_takes():
    from tokensprint_b200 import ops

    assert ops.attention_decode_flat_supported(32, 8, 128, 16, 64, 1)
    assert not ops.attention_decode_flat_supported(32, 8, 80, 16, 64, 1)    # head size no multiple of 64
    assert not ops.attention_decode_flat_supported(32, 8, 128, 4, 64, 1)    # pages too small for the copy engine
    assert not ops.attention_decode_flat_supported(32, 8, 128, 16, 64, 5)   # 20 rows per pair
    assert not ops.attention_decode_flat_supported(32, 8, 128, 16, 600, 1)  # too many sequences
    case = finish_case(paged_case([(5, 70)], 32, 8, 128, 16, torch.bfloat16, seed=1))
    with pytest.raises(ops.KernelError, match="at most 16 rows"):
        run_flat(case)


@pytest.mark.parametrize("splits,chunk", [(16, 64), (8, 128), (4, 256), (2, 512), (64, 64)])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(32, 8, 128, 16, 0), (4, 2, 16, 16, 0), (5, 1, 48, 4, 90), (16, 1, 64, 32, 700)])
def test_attention_mma_decode_with_fixed_key_chunks(splits, chunk, nq, nkv, d, page, window):
    """Sequences of very different lengths in one batch; every CTA takes `chunk` keys, CTAs
    beyond a sequence's end do nothing, and the plan from ops covers the longest one."""
    from tokensprint_b200 import ops

    case = finish_case(paged_case(DECODE, nq, nkv, d, page, torch.bfloat16, seed=5 * d))
    got = run_mma(case, window, splits, chunk)
    want = plain_attention(case, window)
    assert rel_err(got, want) < 1e-2
    plan_splits, plan_chunk = ops.attention_decode_plan(len(DECODE), nkv, 1000, d)
    assert plan_splits * max(plan_chunk, 1) >= 1000 or plan_splits == 1
    assert rel_err(run_mma(case, window, plan_splits, plan_chunk), want) < 1e-2


@pytest.mark.parametrize("kernel", ["simple32", "simple16", "mma", "mma_split"])
@pytest.mark.parametrize("target", ["first", "far", "page_edge_before", "page_edge_after", "block_edge", "last", "window_first", "window_out"])
def test_attention_finds_one_key_that_stands_out(kernel, target):
    """One key is made to match the query; its value is a marker.  Whatever position it has
    (the first key of all, a far one among hundreds, either side of a page's edge, the edge of a
    64-key block, the last key, the oldest key inside a window, the newest key outside it), the
    output must be its value, or must not be for the key outside the window."""
    nq, nkv, d, page, ctx = 4, 1, 64, 16, 700
    window = 0
    where = {"first": 0, "far": 3, "page_edge_before": 16 * 20 - 1, "page_edge_after": 16 * 20, "block_edge": 64 * 7,
             "last": ctx - 1}.get(target)
    if target == "window_first":
        window, where = 100, ctx - 100
    if target == "window_out":
        window, where = 100, ctx - 101
    dtype = torch.float32 if kernel == "simple32" else torch.bfloat16
    case = paged_case([(1, ctx)], nq, nkv, d, page, dtype, seed=5)
    q, k, v = case["dense"][0]
    k.mul_(0.05)
    k[where, 0] = q[0, 2] * 3.0  # head 2's query finds itself at `where`
    v[where, 0] = 10.0
    case = finish_case(case)
    if kernel.startswith("simple"):
        got = run_simple(case, window)
    else:
        got = run_mma(case, window, 4 if kernel == "mma_split" else 1)
    head2 = got.view(1, nq, d)[0, 2].float()
    if target == "window_out":
        assert float(head2.abs().max()) < 5.0, "a key outside the window was seen"
    else:
        assert float((head2 - 10.0).abs().max()) < 0.05, f"the key at {where} was not found"
    assert rel_err(got, plain_attention(case, window)) < (3e-6 if dtype == torch.float32 else 1e-2)


def test_attention_ignores_pages_that_are_not_held():
    """Table entries of -1 (pages a window gave back) and NaN in unused pages must not leak."""
    nq, nkv, d, page, ctx, window = 4, 2, 32, 8, 200, 40
    case = finish_case(paged_case([(3, ctx), (1, 90)], nq, nkv, d, page, torch.bfloat16, seed=9))
    want = plain_attention(case, window)
    # give back every page wholly before the window of the first query of each sequence
    for b, (ql, c) in enumerate(case["seqs"]):
        first_needed = max(0, c - ql - window + 1) // page
        for i in range(first_needed):
            pg = int(case["table"][b, i])
            case["kc"][pg] = float("nan")
            case["vc"][pg] = float("nan")
            case["table"][b, i] = -1
    for got in (run_simple(case, window), run_mma(case, window), run_mma(case, window, 3)):
        assert rel_err(got, want) < 1e-2


# ---------------------------------------------------------------------------
# prompt attention on tcgen05 (head size 128)


def run_tcgen05(case, window=0, mode=0):
    from tokensprint_b200 import ops

    out = torch.full_like(case["q"], float("nan"))
    max_q = max(ql for ql, _ in case["seqs"])
    ops.attention_prefill_tcgen05(case["q"], case["kc"], case["vc"], out, case["cu"], case["ctxs"], case["table"],
                                  case["page"], case["B"], max_q, case["nq"], case["nkv"], case["d"] ** -0.5, window, mode)
    torch.cuda.synchronize()
    ops.check_device_errors()
    return out


PROMPTS = [(1, 1), (1, 77), (5, 5), (3, 130), (64, 64), (37, 200), (2, 65), (1, 64), (130, 131), (300, 300), (129, 517), (33, 1000)]


@pytest.mark.parametrize(
    "nq,nkv,page,window",
    [(32, 8, 16, 0), (4, 4, 16, 0), (8, 1, 8, 0), (16, 1, 64, 0), (2, 1, 32, 0), (6, 3, 16, 0), (128, 1, 16, 0),
     (32, 8, 16, 100), (8, 2, 32, 7), (4, 1, 8, 64), (3, 3, 16, 300), (32, 8, 256, 0), (8, 2, 128, 90), (4, 1, 384, 0),
     (40, 8, 16, 0), (5, 1, 16, 33), (6, 2, 8, 0), (7, 1, 64, 0), (12, 1, 16, 50), (100, 1, 16, 0), (20, 2, 32, 0)],
)
@pytest.mark.parametrize("mode", [1, 2])
def test_attention_tcgen05_mixed(nq, nkv, page, window, mode):
    """Prompt portions and single tokens of many lengths in one launch, group sizes that divide 128
    and group sizes that do not (5: a tile holds 25 tokens and leaves three rows empty; 3, 7, 12,
    100: one token and 28 empty rows), pages of 8 to 256 slots in shuffled order, NaN in every slot
    nobody wrote."""
    case = finish_case(paged_case(PROMPTS, nq, nkv, 128, page, torch.bfloat16, seed=nq + page))
    got = run_tcgen05(case, window, mode)
    want = plain_attention(case, window)
    assert rel_err(got, want) < 1e-2
    assert torch.equal(run_tcgen05(case, window, mode), got)


@pytest.mark.parametrize("mode", [1, 2])
def test_attention_tcgen05_long_context_with_small_pages(mode):
    """More block-table entries than the kernel keeps in shared memory (1,024): the entries
    beyond come straight from the table.  9,000 keys in pages of 8; one portion starts deep inside."""
    case = finish_case(paged_case([(260, 9000), (3, 8300)], 4, 1, 128, 8, torch.bfloat16, seed=21))
    got = run_tcgen05(case, 0, mode)
    assert rel_err(got, plain_attention(case, 0)) < 1e-2


def test_attention_tcgen05_says_what_it_takes():
    from tokensprint_b200 import ops

    assert ops.attention_tcgen05_supported(32, 8, 128, 16)
    assert not ops.attention_tcgen05_supported(32, 8, 64, 16)  # head size
    assert ops.attention_tcgen05_supported(40, 8, 128, 16)  # groups of 5: 25 tokens to a tile
    assert not ops.attention_tcgen05_supported(129, 1, 128, 16)  # more heads to a group than a tile has rows
    assert not ops.attention_tcgen05_supported(32, 8, 128, 4)  # pages too small for one copy each
    assert not ops.attention_tcgen05_supported(32, 8, 128, 96)  # pages that straddle the 64-key blocks
    assert not ops.attention_tcgen05_supported(32, 8, 128, 192)  # and pages that straddle the 128-key blocks of the two-tile kernel
    assert ops.attention_tcgen05_supported(32, 8, 128, 384)
    case = finish_case(paged_case([(5, 9)], 10, 2, 128, 4, torch.bfloat16))
    with pytest.raises(ops.KernelError, match="page size"):
        run_tcgen05(case)


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("target", ["first", "far", "page_edge_before", "page_edge_after", "block_edge", "own", "window_first", "window_out"])
def test_attention_tcgen05_finds_one_key_that_stands_out(target, mode):
    """As for the other kernels, with a prompt portion: the query is token 650 of 700 and the
    portion holds the last 100 tokens."""
    nq, nkv, d, page, ctx, ql = 8, 2, 128, 16, 700, 100
    qpos = 650
    window = 0
    where = {"first": 0, "far": 3, "page_edge_before": 16 * 20 - 1, "page_edge_after": 16 * 20, "block_edge": 64 * 7, "own": qpos}.get(target)
    if target == "window_first":
        window, where = 100, qpos - 99
    if target == "window_out":
        window, where = 100, qpos - 100
    case = paged_case([(7, 40), (ql, ctx)], nq, nkv, d, page, torch.bfloat16, seed=5)
    q, k, v = case["dense"][1]
    k.mul_(0.05)
    qi = qpos - (ctx - ql)
    k[where, 1] = q[qi, 6] * 3.0  # head 6 (KV head 1) of that token finds itself at `where`
    v[where, 1] = 10.0
    case = finish_case(case)
    got = run_tcgen05(case, window, mode)
    row = got.view(-1, nq, d)[7 + qi, 6].float()
    if target == "window_out":
        assert float(row.abs().max()) < 5.0, "a key outside the window was seen"
    else:
        assert float((row - 10.0).abs().max()) < 0.05, f"the key at {where} was not found"
    assert rel_err(got, plain_attention(case, window)) < 1e-2


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("target", ["first", "tile_edge_before", "tile_edge_after", "own"])
def test_attention_tcgen05_groups_of_five_find_one_key_that_stands_out(target, mode):
    """Qwen3-14B's heads (40 over 8): a tile holds 25 tokens, so token 25 of a portion is the first
    row of the second tile.  One query head of one token finds one key, on both sides of that edge."""
    nq, nkv, d, page, ctx, ql = 40, 8, 128, 16, 300, 60
    qi = {"tile_edge_before": 24, "tile_edge_after": 25}.get(target, 40)
    qpos = ctx - ql + qi
    where = {"first": 0, "own": qpos}.get(target, 111)
    case = paged_case([(3, 40), (ql, ctx)], nq, nkv, d, page, torch.bfloat16, seed=6)
    q, k, v = case["dense"][1]
    k.mul_(0.05)
    k[where, 3] = q[qi, 17] * 3.0  # head 17 belongs to KV head 17 // 5 = 3
    v[where, 3] = 10.0
    case = finish_case(case)
    got = run_tcgen05(case, 0, mode)
    row = got.view(-1, nq, d)[3 + qi, 17].float()
    assert float((row - 10.0).abs().max()) < 0.05, f"the key at {where} was not found"
    other = got.view(-1, nq, d)[3 + qi, 12].float()  # a head of KV head 2 does not see it
    assert float(other.abs().max()) < 5.0
    assert rel_err(got, plain_attention(case, 0)) < 1e-2


def test_attention_tcgen05_ignores_pages_that_are_not_held():
    nq, nkv, d, page, window = 8, 2, 128, 8, 40
    case = finish_case(paged_case([(3, 200), (1, 90), (70, 400)], nq, nkv, d, page, torch.bfloat16, seed=9))
    want = plain_attention(case, window)
    for b, (ql, c) in enumerate(case["seqs"]):
        first_needed = max(0, c - ql - window + 1) // page
        for i in range(first_needed):
            pg = int(case["table"][b, i])
            case["kc"][pg] = float("nan")
            case["vc"][pg] = float("nan")
            case["table"][b, i] = -1
    for mode in (1, 2):
        assert rel_err(run_tcgen05(case, window, mode), want) < 1e-2


# ---------------------------------------------------------------------------
# sampling


def test_sample_greedy_and_ties():
    from tokensprint_b200 import ops

    R, V = 5, 1031
    logits = torch.randn(R, V, device=DEV)
    logits[1, 100] = logits[1, 900] = 50.0  # a tie: the lower index wins
    logits[2, V - 1] = 60.0
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits, torch.zeros(R, device=DEV), None, out)
    want = [int(torch.argmax(logits[r])) for r in range(R)]
    want[1] = 100
    assert out.tolist() == want


def test_sample_matches_the_plain_race_and_the_distribution():
    from tokensprint_b200 import ops

    V = 12
    base = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, 3.0, 0.1, 0.2, -3.0, 1.5, 0.7, 0.3])
    R = 4000
    logits = base.repeat(R, 1).to(DEV)
    temps = torch.full((R,), 0.7, device=DEV)
    keys = torch.arange(R, dtype=torch.int64, device=DEV) * 7919 - 1000
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits, temps, keys, out)
    got = out.tolist()
    for r in range(0, 60):
        assert got[r] == plain.sample_token(base, 0.7, int(keys[r]))
    freq = np.bincount(got, minlength=V) / R
    p = torch.softmax(base.double() / 0.7, dim=-1).numpy()
    assert np.abs(freq - p).max() < 4 * np.sqrt(0.25 / R)
    # the same keys give the same tokens; other keys give other tokens
    out2 = torch.empty_like(out)
    ops.sample(logits, temps, keys, out2)
    assert out2.tolist() == got
    ops.sample(logits, temps, keys + 1, out2)
    assert out2.tolist() != got


def test_sample_race_draw_by_draw_on_odd_widths_and_unaligned_rows():
    """Rows that do not start on 16-byte boundaries (a width that is no multiple of four), a
    vocabulary that ends in the middle of a thread's four entries, several chunks: every draw is the
    plain race's draw (the noise of entry i comes from the hash of (key, i // 2))."""
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(17)
    R, V = 24, 4099
    logits = (torch.randn(R, V, generator=g) * 2.0).to(DEV)
    temps = torch.tensor([0.5 + 0.05 * r for r in range(R)], device=DEV)
    keys = (torch.arange(R, dtype=torch.int64) * 104729 - 55).to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits, temps, keys, out)
    for r in range(R):
        assert int(out[r]) == plain.sample_token(logits[r].cpu(), float(temps[r]), int(keys[r])), f"row {r}"
    # a view with a row stride that is larger than the width
    wide = torch.zeros(R, V + 5, device=DEV)
    wide[:, :V] = logits
    out2 = torch.empty_like(out)
    ops.sample(wide[:, :V], temps, keys, out2)
    assert torch.equal(out, out2)


# ---------------------------------------------------------------------------
# skinny GEMM on tcgen05


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize(
    "M,N,K",
    [(1, 128, 64), (8, 6144, 4096), (16, 4096, 12288), (3, 200, 72), (17, 384, 1000), (33, 1000, 4096), (64, 2048, 1024),
     (100, 300, 520), (128, 256, 512), (5, 24576, 1024)],
)
def test_gemm_skinny_tcgen05(M, N, K, out_dtype):
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(DEV, torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    ops.gemm_skinny_bf16(x, w, out)
    torch.cuda.synchronize()
    ops.check_device_errors()
    want = x.double() @ w.double().T
    tol = 1e-2 if out_dtype == torch.bfloat16 else 1e-5
    assert rel_err(out, want) < tol
    # twice in a row (the ticket counters must be back at zero), and a row alone gives the same bits
    out2 = torch.full_like(out, float("nan"))
    ops.gemm_skinny_bf16(x, w, out2)
    assert torch.equal(out, out2)
    out1 = torch.empty((1, N), device=DEV, dtype=out_dtype)
    ops.gemm_skinny_bf16(x[M - 1 :], w, out1)
    assert torch.equal(out1[0], out[M - 1])


@pytest.mark.parametrize("scaled", [False, True])
@pytest.mark.parametrize("M,N,K", [(8, 384, 256), (5, 200, 520), (1, 4096, 4096), (32, 1000, 72), (17, 128, 12288)])
def test_gemm_skinny_fused_row_scale(M, N, K, scaled):
    """Plain output, every row multiplied by the 1/rms that the sums of squares give."""
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(DEV, torch.bfloat16)
    ssq = (torch.rand(3, M, generator=g) * 50 + 1).to(DEV)
    width, eps = 96, 1e-3
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=dtype)
        ops.gemm_skinny_fused(x, w, out=out, scale_ssq=ssq if scaled else None, scale_width=width, scale_eps=eps)
        torch.cuda.synchronize()
        ops.check_device_errors()
        want = x.double() @ w.double().T
        if scaled:
            want = want * torch.rsqrt(ssq.double().sum(0) / width + eps)[:, None]
        assert rel_err(out, want) < (1e-2 if dtype == torch.bfloat16 else 1e-5)
        out2 = torch.full_like(out, float("nan"))
        ops.gemm_skinny_fused(x, w, out=out2, scale_ssq=ssq if scaled else None, scale_width=width, scale_eps=eps)
        assert torch.equal(out, out2)


@pytest.mark.parametrize("M,I,K", [(8, 192, 256), (3, 64, 1032), (32, 12288, 4096), (1, 1024, 4096)])
def test_gemm_skinny_fused_swiglu(M, I, K):
    """Gate and up rows stacked in blocks of 64 + 64: the activation comes out of the GEMM."""
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    gate = (torch.randn(I, K, generator=g) * 0.05).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g) * 0.05).to(torch.bfloat16)
    stacked = torch.stack([gate.view(I // 64, 64, K), up.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous().to(DEV)
    ssq = (torch.rand(2, M, generator=g) * 5 + 1).to(DEV)
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_skinny_fused(x, stacked, out=out, mode=ops.GEMM_EPILOGUE_SWIGLU, scale_ssq=ssq, scale_width=K, scale_eps=1e-6)
    torch.cuda.synchronize()
    ops.check_device_errors()
    r = torch.rsqrt(ssq.double().sum(0) / K + 1e-6)[:, None].cpu()
    gd, ud = (x.double().cpu() @ gate.double().T) * r, (x.double().cpu() @ up.double().T) * r
    want = gd * torch.sigmoid(gd) * ud
    assert rel_err(out, want) < 1e-2
    out2 = torch.full_like(out, float("nan"))
    ops.gemm_skinny_fused(x, stacked, out=out2, mode=ops.GEMM_EPILOGUE_SWIGLU, scale_ssq=ssq, scale_width=K, scale_eps=1e-6)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("M,N,K", [(8, 384, 256), (5, 200, 520), (2, 4096, 12288), (32, 4096, 4096), (7, 100, 64), (3, 202, 64), (20, 99, 128), (17, 131, 72)])
def test_gemm_skinny_fused_residual_and_norm_input(M, N, K):
    """hidden += product, the next norm's input (without its 1/rms) and the sums of squares that
    give the 1/rms, all from the GEMM; then a second GEMM uses them and matches norm + product."""
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(DEV, torch.bfloat16)
    hidden0 = torch.randn(M, N, generator=g).to(DEV)
    norm_w = (1 + 0.1 * torch.randn(N, generator=g)).to(DEV)
    hidden = hidden0.clone()
    xprime = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    tiles = -(-N // 128)
    ssq = torch.full((tiles, M), float("nan"), device=DEV)
    ops.gemm_skinny_fused(x, w, mode=ops.GEMM_EPILOGUE_RESIDUAL_NORM, hidden=hidden, norm_weight=norm_w, xprime=xprime, ssq_out=ssq)
    torch.cuda.synchronize()
    ops.check_device_errors()
    want_h = hidden0.double() + x.double() @ w.double().T
    assert rel_err(hidden, want_h) < 1e-5
    assert rel_err(xprime, want_h * norm_w.double()) < 1e-2
    assert rel_err(ssq.sum(0), (want_h**2).sum(1)) < 1e-5
    # the same again gives the same bits (one writer per tile, sums in a fixed order)
    hidden_b, xprime_b, ssq_b = hidden0.clone(), torch.empty_like(xprime), torch.empty_like(ssq)
    ops.gemm_skinny_fused(x, w, mode=ops.GEMM_EPILOGUE_RESIDUAL_NORM, hidden=hidden_b, norm_weight=norm_w, xprime=xprime_b, ssq_out=ssq_b)
    assert torch.equal(hidden, hidden_b) and torch.equal(xprime, xprime_b) and torch.equal(ssq, ssq_b)
    # consumer: a product with the normed rows
    if N % 8 == 0:
        eps = 1e-5
        w2 = (torch.randn(136, N, generator=g) * 0.05).to(DEV, torch.bfloat16)
        out = torch.empty((M, 136), device=DEV, dtype=torch.float32)
        ops.gemm_skinny_fused(xprime, w2, out=out, scale_ssq=ssq, scale_width=N, scale_eps=eps)
        normed = want_h * torch.rsqrt((want_h**2).mean(1, keepdim=True) + eps) * norm_w.double()
        assert rel_err(out, normed @ w2.double().T) < 1e-2


@pytest.mark.parametrize("M,nq,nkv,K,rope,norm", [(8, 32, 8, 4096, True, True), (3, 4, 2, 256, True, False), (32, 2, 1, 520, False, True), (5, 8, 8, 1024, True, True)])
def test_gemm_skinny_qk_rope_store(M, nq, nkv, K, rope, norm):
    """The q/k/v projection with per-head norm, rotation and the cache store in its epilogue,
    against the projection followed by the kernel that does the same on its own."""
    from tokensprint_b200 import ops

    d = 128
    g = torch.Generator().manual_seed(M + nq + K)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    w = (torch.randn((nq + 2 * nkv) * d, K, generator=g) * 0.05).to(DEV, torch.bfloat16)
    qw = (1 + 0.2 * torch.randn(d, generator=g)).to(DEV) if norm else None
    kw = (1 + 0.2 * torch.randn(d, generator=g)).to(DEV) if norm else None
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, d, 2).float() / d))).to(DEV) if rope else None
    positions = torch.randint(0, 3000, (M,), generator=g).to(DEV, torch.int32)
    slots = torch.randperm(M + 7, generator=g)[:M].to(DEV, torch.int32)
    slots[M // 2] = -1  # a row whose key and value are not stored
    ssq = (torch.rand(2, M, generator=g) * 5 + 1).to(DEV)

    def caches():
        return torch.full((M + 7, nkv, d), 7.0, device=DEV, dtype=torch.bfloat16), torch.full((M + 7, nkv, d), 7.0, device=DEV, dtype=torch.bfloat16)

    # reference: float64 product with the row scale, then the plain functions
    r = torch.rsqrt(ssq.double().sum(0) / K + 1e-6)[:, None].cpu()
    qkv = (x.double().cpu() @ w.double().cpu().T) * r
    heads = qkv.view(M, nq + 2 * nkv, d)
    qh, kh, vh = heads[:, :nq], heads[:, nq : nq + nkv], heads[:, nq + nkv :]
    if norm:
        qh = plain.rms_norm(qh, qw.double().cpu(), 1e-5)
        kh = plain.rms_norm(kh, kw.double().cpu(), 1e-5)
    if rope:
        ang = plain.rope_angles(positions.tolist(), d, 1e4)
        qh, kh = plain.apply_rope(qh, ang), plain.apply_rope(kh, ang)

    q = torch.full((M, nq * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    kc, vc = caches()
    ops.gemm_qk_rope_store(x, w, q, kc, vc, slots, positions, qw, kw, 1e-5, inv_freq, nq, nkv, scale_ssq=ssq, scale_width=K, scale_eps=1e-6)
    torch.cuda.synchronize()
    ops.check_device_errors()
    assert rel_err(q.view(M, nq, d), qh) < 1e-2
    for m in range(M):
        s_ = int(slots[m])
        if s_ >= 0:
            assert rel_err(kc[s_], kh[m]) < 1e-2 and rel_err(vc[s_], vh[m]) < 1e-2
    used = {int(v) for v in slots.tolist() if v >= 0}
    for s_ in range(M + 7):
        if s_ not in used:
            assert bool((kc[s_] == 7.0).all()) and bool((vc[s_] == 7.0).all()), "a slot nobody owns was written"
    q2, (kc2, vc2) = torch.empty_like(q), caches()
    ops.gemm_qk_rope_store(x, w, q2, kc2, vc2, slots, positions, qw, kw, 1e-5, inv_freq, nq, nkv, scale_ssq=ssq, scale_width=K, scale_eps=1e-6)
    assert torch.equal(q, q2) and torch.equal(kc, kc2) and torch.equal(vc, vc2)
    if rope:
        # with the step's table of cosines and sines instead of the epilogue's own: the same bits
        table = ops.rope_cos_sin(positions, inv_freq, M)
        want = torch.stack([torch.cos(positions.float()[:, None] * inv_freq[None, :]), torch.sin(positions.float()[:, None] * inv_freq[None, :])], dim=-1)
        assert table.shape == (M, d // 2, 2) and float((table - want).abs().max()) < 2e-6
        q3, (kc3, vc3) = torch.empty_like(q), caches()
        ops.gemm_qk_rope_store(x, w, q3, kc3, vc3, slots, positions, qw, kw, 1e-5, inv_freq, nq, nkv, scale_ssq=ssq, scale_width=K, scale_eps=1e-6,
                               cos_sin=table)
        assert torch.equal(q, q3) and torch.equal(kc, kc3) and torch.equal(vc, vc3)
        with pytest.raises(ops.KernelError, match="cos_sin"):
            ops.gemm_qk_rope_store(x, w, q3, kc3, vc3, slots, positions, qw, kw, 1e-5, inv_freq, nq, nkv, cos_sin=table[: M - 1] if M > 1 else table.half())


def test_gemm_skinny_refuses_what_it_cannot_take():
    from tokensprint_b200 import ops

    x = torch.zeros(129, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError):
        ops.gemm_skinny_bf16(x, w, torch.empty(129, 128, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ops.KernelError):
        ops.gemm_skinny_bf16(x[:4, :60], w[:, :60], torch.empty(4, 128, device=DEV, dtype=torch.bfloat16))
    # a weight of 2^31 or more (128-row tile x 64-wide chunk) units: the kernel counts them in 32 bits and the entry
    # point says so before anything is read (the pointers are of small buffers: nothing may touch them)
    scratch = torch.zeros(4096, device=DEV)
    counters = torch.zeros(4096, device=DEV, dtype=torch.int32)
    error = torch.zeros(1, device=DEV, dtype=torch.int32)
    N, K = 1 << 27, 1 << 17
    status = ops._fn("ts_gemm_skinny_bf16")(x.data_ptr(), w.data_ptr(), scratch.data_ptr(), 1, N, K, K, K, N, 0,
                                            scratch.data_ptr(), counters.data_ptr(), error.data_ptr(), None, 0, None)
    assert status == -2  # TS_ERR_UNSUPPORTED_SIZE
    torch.cuda.synchronize()
    assert int(error.item()) == 0 and int(counters.abs().sum()) == 0


def test_kernel_bench_runs_a_small_case(capsys):
    """The kernel table's program, on its smallest decode-attention case: one line per kernel with a
    time and a share of the roofline."""
    import json

    from tokensprint_b200 import kernel_bench

    assert kernel_bench.main(["--only", "decode", "--batches", "2", "--contexts", "256", "--json"]) == 0
    rows = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert [r["kernel"] for r in rows] == ["attention, decode", "attention, decode, even shares"]
    assert all(r["us"] > 0 and 0 < r["frac"] < 1.5 and r["unit"] == "GB/s" for r in rows)


def test_feed_tokens():
    from tokensprint_b200 import ops

    ids = torch.arange(100, 120, dtype=torch.int32, device=DEV)
    source = torch.tensor([7, 8, 9, 10], dtype=torch.int32, device=DEV)
    lanes = torch.tensor([3, 0, 19, 5, 5, 5], dtype=torch.int32, device=DEV)
    rows = torch.tensor([2, 0, 3, 1, 1, 1], dtype=torch.int32, device=DEV)
    ops.feed_tokens(ids, source, lanes, rows, 3)  # only the first three pairs
    want = list(range(100, 120))
    want[3], want[0], want[19] = 9, 7, 10
    assert ids.tolist() == want
    ops.feed_tokens(ids, source, lanes, rows, 0)
    assert ids.tolist() == want
    with pytest.raises(ops.KernelError, match="index arrays hold"):
        ops.feed_tokens(ids, source, lanes, rows, 7)


def test_a_wait_that_runs_out_becomes_an_exception_and_the_next_launch_is_clean():
    """The give-up path of the bounded waits: a kernel whose only wait is on an mbarrier that
    nothing feeds runs out of tries (a few thousand), raises the error word as the tcgen05 kernels
    do and returns; the host turns the word into a KernelError, clears it, and the stream goes on
    working.  Nothing faults, traps or hangs."""
    from tokensprint_b200 import ops

    torch.cuda.synchronize()
    ops.check_device_errors()  # nothing pending
    ops.wait_gives_up_probe(torch.device(DEV), limit=4096)
    torch.cuda.synchronize()
    with pytest.raises(ops.KernelError, match="gave up"):
        ops.check_device_errors()
    ops.check_device_errors()  # the word was cleared
    x = torch.randn(8, 256, device=DEV).to(torch.bfloat16)
    w = torch.randn(384, 256, device=DEV).to(torch.bfloat16)
    out = torch.empty(8, 384, device=DEV, dtype=torch.bfloat16)
    ops.gemm_skinny_bf16(x, w, out)
    torch.cuda.synchronize()
    ops.check_device_errors()
    want = x.float() @ w.float().T
    assert float((out.float() - want).abs().max()) <= 2e-2 * float(want.abs().max())


def _layer_like_products(ops, M, H, I, nq, nkv, tensors):
    """The four products between two attention kernels of a decode step: the output projection
    (into the residual stream, preparing the next norm), gate/up with the activation, down (into the
    residual stream again), and the next layer's q/k/v projection with norm, rotation and cache
    store.  Returns everything they wrote."""
    t = tensors
    d = 128
    hidden = t["hidden0"].clone()
    x1 = torch.empty((M, H), device=DEV, dtype=torch.bfloat16)
    ssq1 = torch.empty((-(-H // 128), M), device=DEV)
    ops.gemm_skinny_fused(t["attn"], t["wo"], mode=ops.GEMM_EPILOGUE_RESIDUAL_NORM, hidden=hidden, norm_weight=t["n1"], xprime=x1, ssq_out=ssq1)
    act = torch.empty((M, I), device=DEV, dtype=torch.bfloat16)
    ops.gemm_skinny_fused(x1, t["wgu"], out=act, mode=ops.GEMM_EPILOGUE_SWIGLU, scale_ssq=ssq1, scale_width=H, scale_eps=1e-6)
    x2 = torch.empty((M, H), device=DEV, dtype=torch.bfloat16)
    ssq2 = torch.empty((-(-H // 128), M), device=DEV)
    ops.gemm_skinny_fused(act, t["wd"], mode=ops.GEMM_EPILOGUE_RESIDUAL_NORM, hidden=hidden, norm_weight=t["n2"], xprime=x2, ssq_out=ssq2)
    q = torch.empty((M, nq * d), device=DEV, dtype=torch.bfloat16)
    kc, vc = torch.zeros_like(t["kc"]), torch.zeros_like(t["kc"])
    ops.gemm_qk_rope_store(x2, t["wqkv"], q, kc, vc, t["slots"], t["pos"], t["qn"], t["kn"], 1e-6, t["inv_freq"], nq, nkv,
                           scale_ssq=ssq2, scale_width=H, scale_eps=1e-6)
    return {"hidden": hidden, "x1": x1, "ssq1": ssq1, "act": act, "x2": x2, "ssq2": ssq2, "q": q, "kc": kc, "vc": vc}


@pytest.mark.parametrize("M,H,I,nq,nkv", [(8, 1024, 3072, 16, 8), (1, 4096, 12288, 32, 8), (32, 640, 1408, 5, 1), (17, 5120, 1024, 40, 8)])
def test_gemm_chain_launches_products_together_and_changes_no_bit(M, H, I, nq, nkv):
    """Four products that feed one another, once each as a launch of its own and once inside a chain
    (one kernel: each phase starts fetching its weights while the one before is being finished, and
    reads its inputs after a barrier over the grid): the same bits, twice in a row, and the float64
    result within bfloat16 rounding."""
    from tokensprint_b200 import ops

    d = 128
    g = torch.Generator().manual_seed(M * 7 + H)
    bf = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(DEV, torch.bfloat16)
    gate, up = bf(I, H, s=0.03), bf(I, H, s=0.03)
    t = {
        "attn": bf(M, nq * d), "wo": bf(H, nq * d, s=0.03), "wd": bf(H, I, s=0.03), "wqkv": bf((nq + 2 * nkv) * d, H, s=0.03),
        "wgu": torch.stack([gate.view(I // 64, 64, H), up.view(I // 64, 64, H)], dim=1).reshape(2 * I, H).contiguous(),
        "hidden0": torch.randn(M, H, generator=g).to(DEV), "n1": (1 + 0.1 * torch.randn(H, generator=g)).to(DEV),
        "n2": (1 + 0.1 * torch.randn(H, generator=g)).to(DEV), "qn": (1 + 0.1 * torch.randn(d, generator=g)).to(DEV),
        "kn": (1 + 0.1 * torch.randn(d, generator=g)).to(DEV), "inv_freq": plain.rope_inverse_frequencies(d, 1e6).to(DEV),
        "kc": torch.zeros(64, nkv, d, device=DEV, dtype=torch.bfloat16),
        "slots": torch.randperm(64, generator=g)[:M].to(DEV, torch.int32), "pos": torch.randint(0, 3000, (M,), generator=g).to(DEV, torch.int32),
    }
    one_by_one = _layer_like_products(ops, M, H, I, nq, nkv, t)
    torch.cuda.synchronize()
    for _ in range(2):
        before = ops.launch_count
        with ops.gemm_chain(torch.device(DEV)):
            chained = _layer_like_products(ops, M, H, I, nq, nkv, t)
        assert ops.launch_count - before == 1, "the four products were not one launch"
        torch.cuda.synchronize()
        ops.check_device_errors()
        for name, want in one_by_one.items():
            assert torch.equal(chained[name], want), f"{name} differs between the chain and single launches"
    # and the arithmetic itself
    h1 = t["hidden0"].double() + t["attn"].double() @ t["wo"].double().T
    assert rel_err(one_by_one["x1"], h1 * t["n1"].double()) < 1e-2
    n1 = (h1 * torch.rsqrt((h1**2).mean(1, keepdim=True) + 1e-6) * t["n1"].double())
    gd, ud = n1 @ gate.double().T, n1 @ up.double().T
    assert rel_err(one_by_one["act"], gd * torch.sigmoid(gd) * ud) < 3e-2
    h2 = h1 + one_by_one["act"].double() @ t["wd"].double().T
    assert rel_err(one_by_one["hidden"], h2) < 1e-3
    # six products in one chain: the list holds four, so two launches; any other op launches what is pending
    square = (torch.randn(256, 256, generator=g) * 0.06).to(DEV, torch.bfloat16)
    x0 = (torch.randn(M, 256, generator=g)).to(DEV, torch.bfloat16)

    def six(x):
        for _ in range(6):
            out = torch.empty((M, 256), device=DEV, dtype=torch.bfloat16)
            ops.gemm_skinny_bf16(x, square, out)
            x = out
        return x

    want = six(x0)
    before = ops.launch_count
    with ops.gemm_chain(torch.device(DEV)):
        got = six(x0)
        assert ops.launch_count - before == 1  # the first four went when the fifth arrived
        ids = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.feed_tokens(ids, ids, ids, ids, 0)  # not a product: the two that waited are launched first
        assert ops.launch_count - before == 3
    torch.cuda.synchronize()
    ops.check_device_errors()
    assert torch.equal(got, want)


def test_sample_noise_is_uniform_over_a_large_vocabulary_with_one_key():
    """One key, flat logits, many entries: the winner's index is uniform over the vocabulary, so over
    many draws (keys that differ in one bit each) the winners spread evenly over 16 ranges of indices,
    and neighbouring entries (which share a hash) win equally often."""
    from tokensprint_b200 import ops

    R, V = 4096, 40000
    logits = torch.zeros(R, V, device=DEV)
    temps = torch.ones(R, device=DEV)
    keys = torch.tensor([plain._mix64(7) ^ (1 << (i % 64)) ^ (i // 64) for i in range(R)], dtype=torch.uint64).view(torch.int64).to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits, temps, keys, out)
    got = out.cpu().numpy()
    counts = np.bincount(got * 16 // V, minlength=16)
    assert np.abs(counts - R / 16).max() < 5 * np.sqrt(R / 16), f"winners are not spread evenly: {counts.tolist()}"
    odd = int((got % 2).sum())
    assert abs(odd - R / 2) < 5 * np.sqrt(R / 4), f"odd entries won {odd} of {R} draws"

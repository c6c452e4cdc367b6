"""The allocation-free entry point of the attention library, called through its exported C symbol.

`ts_attention_paged_mma_noalloc` is for callers that cannot allocate device memory (a host
program that embeds the kernel without torch's allocator, a process whose memory has been
handed out in full to other pools, a loop that must stay off the allocator's locks): the
scratch of the split-key decode path lives in the library itself.  The test calls the
symbol with ctypes, twice in a row, a large batch with many key splits and then a small one
with few, so that partial results of another shape lie in the shared array when the second
call runs.  Both calls are made so that the partial results really pass through the array
(the merge inside a thread-block cluster is switched off for one pair of calls, and another
pair uses more splits than a cluster takes); each result is compared with the plain
attention of tests/plain and with the entry point that takes scratch from the caller.  A
batch beyond the built-in scratch must be refused with its own error code.  This file is
collected last on purpose: it must pass alone in a fresh process and after every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

HEAD_DIM = 64


def _library():
    from tokensprint_b200.csrc import build

    lib = build.load_variant("attention_mma", {"TS_HEAD_DIM": HEAD_DIM})
    p, i, f, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    lib.ts_attention_paged_mma.argtypes = [p] * 9 + [i] * 7 + [f, i, i, p]
    lib.ts_attention_paged_mma.restype = i
    lib.ts_attention_paged_mma_noalloc.argtypes = [p] * 8 + [i] * 7 + [f, i, i, p]
    lib.ts_attention_paged_mma_noalloc.restype = i
    lib.ts_attention_noalloc_scratch_floats.restype = ll
    lib.ts_attention_mma_scratch_floats.argtypes = [ll, i]
    lib.ts_attention_mma_scratch_floats.restype = ll
    lib.ts_attention_noalloc_error_text.argtypes = [i]
    lib.ts_attention_noalloc_error_text.restype = ctypes.c_char_p
    return lib


def _batch(contexts, nq, nkv, page, seed):
    """A decode batch: one query token per sequence, keys and values in shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    B = len(contexts)
    blocks = [-(-c // page) for c in contexts]
    pages = sum(blocks) + 2
    order = torch.randperm(pages, generator=g)
    table = torch.full((B, max(blocks)), -1, dtype=torch.int32)
    used = 0
    for b, n in enumerate(blocks):
        table[b, :n] = order[used : used + n].to(torch.int32)
        used += n
    dev = "cuda"
    return dict(
        B=B, nq=nq, nkv=nkv, page=page,
        q=torch.randn(B, nq * HEAD_DIM, generator=g).to(dev, torch.bfloat16),
        kc=torch.randn(pages, page, nkv, HEAD_DIM, generator=g).to(dev, torch.bfloat16),
        vc=torch.randn(pages, page, nkv, HEAD_DIM, generator=g).to(dev, torch.bfloat16),
        table=table.to(dev),
        cu=torch.arange(B + 1, dtype=torch.int32, device=dev),
        ctx=torch.tensor(contexts, dtype=torch.int32, device=dev),
        seq_index=torch.arange(B, dtype=torch.int32, device=dev),
    )


def _call(lib, case, splits, noalloc):
    out = torch.full_like(case["q"], float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    tail = (case["table"].shape[1], case["page"], case["B"], case["B"], 1, case["nq"], case["nkv"],
            HEAD_DIM ** -0.5, 0, splits, stream)
    head = (case["q"].data_ptr(), case["kc"].data_ptr(), case["vc"].data_ptr(), out.data_ptr())
    rest = (case["cu"].data_ptr(), case["ctx"].data_ptr(), case["table"].data_ptr(), case["seq_index"].data_ptr())
    if noalloc:
        status = lib.ts_attention_paged_mma_noalloc(*head, *rest, *tail)
    else:
        n = lib.ts_attention_mma_scratch_floats(case["B"] * case["nq"], splits)
        scratch = torch.full((max(int(n), 1),), float("nan"), device="cuda")
        status = lib.ts_attention_paged_mma(*head, scratch.data_ptr(), *rest, *tail)
    torch.cuda.synchronize()
    return status, out


def _plain(case):
    """Float64 attention of the batch's single query per sequence over all its keys."""
    from tests.plain import qwen3_plain as plain

    kc, vc = case["kc"].double().cpu(), case["vc"].double().cpu()
    table, ctx = case["table"].cpu(), case["ctx"].cpu().tolist()
    page, nq, nkv = case["page"], case["nq"], case["nkv"]
    rows = []
    for b, n in enumerate(ctx):
        pages = table[b, : -(-n // page)].long()
        k = kc[pages].reshape(-1, nkv, HEAD_DIM)[:n]
        v = vc[pages].reshape(-1, nkv, HEAD_DIM)[:n]
        q = torch.zeros(n, nq, HEAD_DIM, dtype=torch.float64)
        q[-1] = case["q"][b].double().cpu().view(nq, HEAD_DIM)
        rows.append(plain.causal_attention(q, k, v, scale=HEAD_DIM ** -0.5)[-1].reshape(-1))
    return torch.stack(rows)


# (contexts, query heads, KV heads, key splits, seed): the larger call first
PAIR_FEW_SPLITS = [([700, 64, 65, 1, 333, 129], 8, 2, 6, 1), ([90, 257], 4, 4, 3, 2)]
PAIR_MANY_SPLITS = [([900, 640, 65, 1, 777, 129, 1000], 8, 2, 12, 3), ([600, 257], 4, 4, 9, 4)]


def _check_pair(lib, pair):
    for contexts, nq, nkv, splits, seed in pair:
        case = _batch(contexts, nq, nkv, 16, seed)
        status, got = _call(lib, case, splits, noalloc=True)
        assert status == 0, lib.ts_attention_noalloc_error_text(status).decode()
        assert torch.isfinite(got.float()).all()
        want = _plain(case)
        err = float((got.double().cpu() - want).abs().max() / want.abs().max())
        assert err < 1e-2, f"no-alloc entry point differs from the plain attention by {err} ({splits} splits)"
        status, other = _call(lib, case, splits, noalloc=False)
        assert status == 0
        err = float((got.float() - other.float()).abs().max() / other.float().abs().max())
        assert err < 1e-2, f"no-alloc entry point differs from the caller-scratch one by {err}"
    return case


def test_noalloc_entry_point_matches_plain_attention_twice_in_a_row():
    lib = _library()
    assert lib.ts_attention_noalloc_scratch_floats() == 2 * 1024 * 1024
    lib.ts_attention_mma_set_cluster_merge.argtypes = [ctypes.c_int]
    before = lib.ts_attention_mma_cluster_merge()
    try:
        # 2..8 splits would merge inside a cluster and never touch the array: switch that off
        lib.ts_attention_mma_set_cluster_merge(0)
        _check_pair(lib, PAIR_FEW_SPLITS)
    finally:
        lib.ts_attention_mma_set_cluster_merge(before)
    # more splits than a cluster takes: through the array whatever the switch says
    case = _check_pair(lib, PAIR_MANY_SPLITS)
    # without key splits no scratch is touched at all
    status, got = _call(lib, case, 1, noalloc=True)
    status2, want = _call(lib, case, 1, noalloc=False)
    assert status == 0 and status2 == 0 and torch.equal(got, want)


def test_noalloc_entry_point_refuses_what_its_scratch_cannot_hold():
    lib = _library()
    limit = lib.ts_attention_noalloc_scratch_floats()
    B, nq, splits = 600, 32, 4
    assert lib.ts_attention_mma_scratch_floats(B * nq, splits) > limit
    case = _batch([40] * B, nq, 8, 16, 3)
    status, _ = _call(lib, case, splits, noalloc=True)
    assert status == -3
    assert b"scratch" in lib.ts_attention_noalloc_error_text(status)
    # the same batch fits with fewer splits or through the other entry point
    status, got = _call(lib, case, 1, noalloc=True)
    status2, want = _call(lib, case, splits, noalloc=False)
    assert status == 0 and status2 == 0
    assert float((got.float() - want.float()).abs().max() / want.float().abs().max()) < 1e-2

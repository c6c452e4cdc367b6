"""Times the engine's kernels one at a time, at the layer sizes of a named preset and over a
range of batch sizes and context lengths, and prints each one's share of its roofline.

    python -m tokensprint_b200.kernel_bench [--preset qwen3-8b] [--only decode,prompt,gemm,small,layer]

Every kernel runs after a read of a buffer larger than the L2 cache, so it reads its operands
from device memory as it does inside a model step, and is timed on the device inside a CUDA graph,
so the host's launch cost is not in the figure.  The denominators are the measured peaks where a
file of them is given, else the fallback figures (named in the output).  Kernels inside a step
overlap their neighbours (they are resident and prefetch before the previous kernel ends), so
these isolated times are upper bounds of what the step pays.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from . import ops
from .config.registry import get_model_config

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks(path: str | None) -> tuple[dict, str]:
    if path and os.path.exists(path):
        with open(path) as f:
            got = json.load(f)
        if "hbm_gbs" in got and "bf16_tflops" in got:
            return {"hbm_gbs": float(got["hbm_gbs"]), "bf16_tflops": float(got["bf16_tflops"])}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class Timer:
    """Device time of one call, with a cold L2 and without the host's launch cost: the call is
    captured in a CUDA graph `reps` times, each after a read of a buffer twice the L2's size (a
    read, so that the L2 is left full of clean lines, as the weights leave it in a model step: after
    a write the kernel would also pay for the write-back of what it evicts); the same graph with
    the reads alone is timed too, and the difference divided by `reps` is the figure (the best of
    a few replays)."""

    def __init__(self, device, reps: int = 8, replays: int = 5):
        self.flush = torch.zeros(64 << 20, dtype=torch.int32, device=device)  # 256 MB
        self.reps, self.replays = reps, replays
        self.stream = torch.cuda.Stream(device)
        self.base = self._time(lambda: None)

    def _time(self, fn) -> float:
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()  # the inputs were made on the caller's stream
        with torch.cuda.stream(self.stream):
            for _ in range(2):
                fn()
            self.stream.synchronize()
            with torch.cuda.graph(graph, stream=self.stream):
                for _ in range(self.reps):
                    self.flush.max()
                    fn()
            best = None
            for _ in range(self.replays):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                graph.replay()
                e1.record(self.stream)
                e1.synchronize()
                t = e0.elapsed_time(e1) * 1e3
                best = t if best is None else min(best, t)
        return best

    def __call__(self, fn) -> float:
        """Microseconds of one call of fn."""
        return max(0.0, self._time(fn) - self.base) / self.reps

    def whole_graph(self, body) -> float:
        """Microseconds of `body` (a sequence of launches that defeats the L2 by itself) captured as
        one graph: the best of a few replays."""
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.stream(self.stream):
            body()
            self.stream.synchronize()
            with torch.cuda.graph(graph, stream=self.stream):
                body()
            best = None
            for _ in range(self.replays):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                graph.replay()
                e1.record(self.stream)
                e1.synchronize()
                t = e0.elapsed_time(e1) * 1e3
                best = t if best is None else min(best, t)
        return best


def _paged(B: int, ctx: int, nkv: int, d: int, page: int, device):
    blocks = -(-ctx // page)
    pages = B * blocks
    k = torch.randn(pages, page, nkv, d, device=device).bfloat16()
    v = torch.randn(pages, page, nkv, d, device=device).bfloat16()
    table = torch.randperm(pages, device=device).int().view(B, blocks).contiguous()
    return k, v, table


def decode_attention(cfg, timer, pk, rows, device, batches=(1, 8, 64), contexts=(1024, 4096, 16384, 32768)):
    nq, nkv, d, page = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, 16
    for B in batches:
        for ctx in contexts:
            if B * ctx * nkv * d * 4 > (24 << 30):
                continue
            k, v, table = _paged(B, ctx, nkv, d, page, device)
            q = torch.randn(B, nq * d, device=device).bfloat16()
            out = torch.empty_like(q)
            cu = torch.arange(B + 1, dtype=torch.int32, device=device)
            lens = torch.full((B,), ctx, dtype=torch.int32, device=device)
            seq_index = torch.arange(B, dtype=torch.int32, device=device)
            gb = B * ctx * nkv * d * 2 * 2 / 1e9
            # the engine plans the split count for a context of at most 2,048 keys (one captured
            # graph serves every length); each sequence then divides its own keys evenly
            splits = ops.attention_decode_splits(B, nkv, min(ctx, 2048), d)
            scratch = torch.empty(ops.attention_scratch_floats(B * nq, splits, d), dtype=torch.float32, device=device) if splits > 1 else None

            def run():
                ops.attention_paged_mma(q, k, v, out, cu, lens, table, seq_index, page, B, 1, nq, nkv, d, d ** -0.5, 0, splits, scratch, 0)

            us = timer(run)
            rows.append(("attention, decode", f"B={B} ctx={ctx} splits={splits}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))
            if ops.attention_decode_flat_supported(nq, nkv, d, page, B, 1):
                def run_flat():
                    ops.attention_decode_flat(q, k, v, out, cu, lens, table, seq_index, page, B, 1, nq, nkv, d, d ** -0.5, 0)

                us = timer(run_flat)
                rows.append(("attention, decode, even shares", f"B={B} ctx={ctx}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))
            del k, v
    ops.check_device_errors()


def prompt_attention(cfg, timer, pk, rows, device):
    nq, nkv, d, page = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, 16
    if not ops.attention_tcgen05_supported(nq, nkv, d, page):
        return
    # (sequences, new tokens of each, keys of each): whole prompts, and a portion at the end of a longer one
    for B, T, ctx in ((8, 256, 256), (1, 2048, 2048), (4, 2048, 2048), (1, 8192, 8192), (1, 2048, 8192), (1, 2048, 32768), (1, 32768, 32768)):
        k, v, table = _paged(B, ctx, nkv, d, page, device)
        q = torch.randn(B * T, nq * d, device=device).bfloat16()
        out = torch.empty_like(q)
        cu = torch.arange(0, B * T + 1, T, dtype=torch.int32, device=device)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=device)

        def run():
            ops.attention_prefill_tcgen05(q, k, v, out, cu, lens, table, page, B, T, nq, nkv, d ** -0.5, 0)

        us = timer(run)
        pairs = B * (T * (ctx - T) + T * (T + 1) / 2)  # (query, key) pairs under the causal mask
        tf = 4 * pairs * nq * d / 1e12
        rows.append(("attention, prompt", f"B={B} new={T} keys={ctx}", us, tf / (us * 1e-6), "TFLOP/s", tf / (us * 1e-6) / pk["bf16_tflops"]))
        del k, v, q, out
    ops.check_device_errors()


def skinny_gemm(cfg, timer, pk, rows, device):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    shapes = (("qkv", (nq + 2 * nkv) * d, H), ("o", H, nq * d), ("gate_up", 2 * I, H), ("down", H, I), ("lm_head", V, H))
    for name, N, K in shapes:
        w = (torch.randn(N, K, device=device) * 0.02).bfloat16()
        for M in (1, 8, 32, 64, 128):
            x = torch.randn(M, K, device=device).bfloat16()
            out = torch.empty(M, N, device=device, dtype=torch.bfloat16)
            if not ops.gemm_skinny_supported(x, w):
                continue
            us = timer(lambda: ops.gemm_skinny_bf16(x, w, out))
            gb = (N * K + M * K + M * N) * 2 / 1e9
            rows.append(("GEMM, few rows", f"{name} M={M} N={N} K={K}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))
        del w
    ops.check_device_errors()


def small_kernels(cfg, timer, pk, rows, device):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    for T in (2048, 8192):
        hidden = torch.randn(T, H, device=device)
        delta = torch.randn(T, H, device=device).bfloat16()
        weight = torch.ones(H, device=device)
        out = torch.empty(T, H, device=device, dtype=torch.bfloat16)
        us = timer(lambda: ops.add_rmsnorm(hidden, delta, weight, out, cfg.rms_norm_eps))
        gb = T * H * (4 + 4 + 2 + 2) / 1e9
        rows.append(("add + RMSNorm", f"T={T} H={H}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))

        gu = torch.randn(T, 2 * I, device=device).bfloat16()
        act = torch.empty(T, I, device=device, dtype=torch.bfloat16)
        us = timer(lambda: ops.swiglu(gu, act))
        gb = T * I * 3 * 2 / 1e9
        rows.append(("SwiGLU", f"T={T} I={I}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))

        page = 16
        pages = T // page
        qkv = torch.randn(T, (nq + 2 * nkv) * d, device=device).bfloat16()
        q = torch.empty(T, nq * d, device=device, dtype=torch.bfloat16)
        kc = torch.empty(pages, page, nkv, d, device=device, dtype=torch.bfloat16)
        vc = torch.empty_like(kc)
        slots = torch.randperm(T, device=device).int()
        pos = torch.arange(T, dtype=torch.int32, device=device)
        qw, kw = torch.ones(d, device=device), torch.ones(d, device=device)
        inv_freq = (cfg.rope_theta ** (-torch.arange(0, d, 2, device=device).float() / d)).contiguous()
        us = timer(lambda: ops.qk_norm_rope_store(qkv, q, kc, vc, slots, pos, qw, kw, cfg.rms_norm_eps, inv_freq, nq, nkv, d))
        gb = T * (nq + 2 * nkv) * d * 2 * 2 / 1e9
        rows.append(("q/k norm + rotation + store", f"T={T}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))

        table = (torch.randn(V, H, device=device) * 0.02).bfloat16()
        ids = torch.randint(0, V, (T,), dtype=torch.int32, device=device)
        us = timer(lambda: ops.embed_gather(hidden, table, ids))
        gb = T * H * (2 + 4) / 1e9
        rows.append(("embedding", f"T={T} V={V}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))
        del table, gu, act, qkv
    for R in (8, 64, 256):
        logits = torch.randn(R, V, device=device)
        temp = torch.full((R,), 0.7, device=device)
        keys = torch.arange(R, dtype=torch.int64, device=device)
        tok = torch.empty(R, dtype=torch.int32, device=device)
        us = timer(lambda: ops.sample(logits, temp, keys, tok))
        gb = R * V * 4 / 1e9
        rows.append(("sampling", f"rows={R} V={V}", us, gb / (us * 1e-6), "GB/s", gb / (us * 1e-6) / pk["hbm_gbs"]))
    ops.check_device_errors()


def layer_products(cfg, timer, pk, rows, device):
    """The four products between two attention kernels of a decode step (output projection into the
    residual stream, gate/up with the activation, down into the residual stream, the next layer's
    q/k/v with norm, rotation and cache store), with all their fused epilogues: once as four
    launches (programmatic dependent launch overlaps their ends and starts), once as one chained
    launch (ops.gemm_chain).  Eight sets of weights take turns, so every launch reads its weights
    from device memory; the figure is a layer's share of a graph of 40 layers."""
    H, I = cfg.hidden_size, cfg.intermediate_size
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    if d != ops.GEMM_QK_ROPE_HEAD_DIM or I % 64:
        return
    sets, reps = 8, 40
    bf = lambda *shape, s=0.03: (torch.randn(*shape, device=device) * s).bfloat16()
    weights = [dict(o=bf(H, nq * d), gu=bf(2 * I, H), down=bf(H, I), qkv=bf((nq + 2 * nkv) * d, H)) for _ in range(sets)]
    layer_bytes = sum(w.numel() * 2 for w in weights[0].values())
    n1, n2 = torch.ones(H, device=device), torch.ones(H, device=device)
    qn, kn = torch.ones(d, device=device), torch.ones(d, device=device)
    inv_freq = (cfg.rope_theta ** (-torch.arange(0, d, 2, device=device).float() / d)).contiguous()
    for M in (1, 8, 32):
        attn, hidden = bf(M, nq * d, s=1.0), torch.randn(M, H, device=device)
        x1, x2 = (torch.empty((M, H), device=device, dtype=torch.bfloat16) for _ in range(2))
        ssq1, ssq2 = (torch.empty((-(-H // 128), M), device=device) for _ in range(2))
        act = torch.empty((M, I), device=device, dtype=torch.bfloat16)
        q = torch.empty((M, nq * d), device=device, dtype=torch.bfloat16)
        kc = torch.zeros(64, nkv, d, device=device, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        slots = torch.arange(M, device=device, dtype=torch.int32)
        pos = torch.arange(M, device=device, dtype=torch.int32)
        cos_sin = ops.rope_cos_sin(pos, inv_freq, M)  # once a step in the engine: not part of a layer

        def layer(w, nxt):
            ops.gemm_skinny_fused(attn, w["o"], mode=ops.GEMM_EPILOGUE_RESIDUAL_NORM, hidden=hidden, norm_weight=n1, xprime=x1, ssq_out=ssq1, prefetch=w["gu"])
            ops.gemm_skinny_fused(x1, w["gu"], out=act, mode=ops.GEMM_EPILOGUE_SWIGLU, scale_ssq=ssq1, scale_width=H, scale_eps=1e-6, prefetch=w["down"])
            ops.gemm_skinny_fused(act, w["down"], mode=ops.GEMM_EPILOGUE_RESIDUAL_NORM, hidden=hidden, norm_weight=n2, xprime=x2, ssq_out=ssq2, prefetch=w["qkv"])
            ops.gemm_qk_rope_store(x2, w["qkv"], q, kc, vc, slots, pos, qn, kn, 1e-6, inv_freq, nq, nkv,
                                   scale_ssq=ssq2, scale_width=H, scale_eps=1e-6, prefetch=nxt["o"], cos_sin=cos_sin)

        for chained in (False, True):
            def body():
                for r in range(reps):
                    if chained:
                        with ops.gemm_chain(device):
                            layer(weights[r % sets], weights[(r + 1) % sets])
                    else:
                        layer(weights[r % sets], weights[(r + 1) % sets])

            us = timer.whole_graph(body) / reps
            gbs = layer_bytes / 1e9 / (us * 1e-6)
            rows.append(("a layer's four products", f"M={M}, {'one chained launch' if chained else 'four launches'}", us, gbs, "GB/s", gbs / pk["hbm_gbs"]))
    ops.check_device_errors()


GROUPS = {"decode": decode_attention, "prompt": prompt_attention, "gemm": skinny_gemm, "small": small_kernels, "layer": layer_products}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--preset", default="qwen3-8b")
    p.add_argument("--only", default=",".join(GROUPS), help="comma-separated groups: " + ", ".join(GROUPS))
    p.add_argument("--peaks", default=os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json"))
    p.add_argument("--batches", default="1,8,64", help="batch sizes of the decode attention cases")
    p.add_argument("--contexts", default="1024,4096,16384,32768", help="context lengths of the decode attention cases")
    p.add_argument("--json", action="store_true", help="one JSON object a row instead of the table")
    args = p.parse_args(argv)
    if not torch.cuda.is_available():
        print("kernel_bench needs a CUDA device", file=sys.stderr)
        return 2
    device = torch.device("cuda:0")
    cfg = get_model_config(args.preset)
    pk, source = peaks(args.peaks)
    timer = Timer(device)
    rows: list[tuple] = []
    for name in args.only.split(","):
        if name not in GROUPS:
            print(f"unknown group {name!r}; known: {', '.join(GROUPS)}", file=sys.stderr)
            return 2
        if name == "decode":
            decode_attention(cfg, timer, pk, rows, device, [int(x) for x in args.batches.split(",")], [int(x) for x in args.contexts.split(",")])
        else:
            GROUPS[name](cfg, timer, pk, rows, device)
    if args.json:
        for kernel, case, us, achieved, unit, frac in rows:
            print(json.dumps({"kernel": kernel, "case": case, "us": round(us, 2), "achieved": round(achieved, 1), "unit": unit, "frac": round(frac, 3), "peaks": source}))
        return 0
    print(f"preset {args.preset}; peaks ({source}): {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s bf16\n")
    print("| kernel | case | us | achieved | of peak |")
    print("|---|---|---|---|---|")
    for kernel, case, us, achieved, unit, frac in rows:
        print(f"| {kernel} | {case} | {us:.1f} | {achieved:.0f} {unit} | {frac:.2f} |")
    return 0


if __name__ == "__main__":
    sys.exit(main())

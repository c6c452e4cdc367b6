"""Python face of the CUDA kernels: argument checks, then one call into the library.

Every function works on CUDA tensors, launches on torch's current stream and returns
without synchronising.  A size that a kernel does not take raises `KernelError` with
the limit in words; nothing falls back to another implementation.
"""

from __future__ import annotations

import ctypes
import os as _os
from typing import Optional

import torch

from tokensprint_b200.csrc import build as _build

DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1}
_GEMM_MAX_TILES = 1 << 16  # size of the ticket-counter arrays of the GEMM and of the decode attention

_c_void_p = ctypes.c_void_p
_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_ll = ctypes.c_longlong

_SIGNATURES = {
    "ts_embed_gather": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "ts_feed_tokens": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p],
    "ts_add_rmsnorm": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
    "ts_residual_add": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "ts_swiglu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "ts_qk_norm_rope_store": [
        _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
        _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
    ],
    "ts_attention_paged_simple": [
        _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p,
    ],
    "ts_sample": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "ts_sgemm_nt": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_void_p],
}

_functions: dict[str, object] = {}


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    return _build.load()


def _fn(name: str):
    f = _functions.get(name)
    if f is None:
        lib = library()
        try:
            f = getattr(lib, name)
        except AttributeError as e:
            raise KernelError(f"the CUDA library has no entry point {name}") from e
        f.argtypes = _SIGNATURES[name]
        f.restype = _c_int
        _functions[name] = f
    return f


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle.  (torch.cuda.current_stream() builds a Python object and
    resolves the device by name every time: a third of the host's time in a step launched kernel by
    kernel; the raw call is a hundred times cheaper.)"""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# Launches of this library's kernels since import (library GEMMs are not counted).
launch_count = 0


def _check(name: str, status: int) -> None:
    global launch_count
    if status == 0:
        launch_count += 1
        return
    if status == -1:
        raise KernelError(f"{name}: bad argument")
    if status == -2:
        raise KernelError(f"{name}: size not supported by this kernel")
    raise KernelError(f"{name}: CUDA error {status} at launch")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _cuda_contig(name: str, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _act_code(name: str, t: torch.Tensor) -> int:
    code = DTYPE_CODES.get(t.dtype)
    if code is None:
        raise KernelError(f"{name} must be float32 or bfloat16, got {t.dtype}")
    return code


# ---------------------------------------------------------------------------
# chains of products: several skinny GEMMs that feed one another, launched as one kernel

# Whether a model step chains its products by itself (Model.chain_scope).  Off: measured on B200 at
# Qwen3-8B sizes, the four products of a decode layer take 87 us as four launches (programmatic
# dependent launch already overlaps a kernel's start with its predecessor's end) and 102 to 109 us
# as one chained launch: what separates two products is the chain of trips to the L2 at the end of
# the first (partial sums, ticket, sums, the finished tile) and the first copies of the second, about
# 8 us either way, and inside one kernel the copies that early CTAs ask for the next phase delay the
# last copies of the late ones.  TS_GEMM_CHAIN=1 switches it on for measurements.
GEMM_CHAIN = _os.environ.get("TS_GEMM_CHAIN", "0") == "1"
_chain_open = False
_chain_keep: list = []  # tensors that products waiting in the chain read or write
_chain_counted = 0


def _chain_sync_words(device: torch.device) -> torch.Tensor:
    """Per (device, stream): the counters of the chained kernel's grid barrier (zero between launches)."""
    counters, _ = _gemm_workspace(device)
    return counters[_GEMM_MAX_TILES:]


class gemm_chain:
    """While this context is open, the engine's own few-row products are not launched when they are
    called: they are collected, and up to `ts_gemm_chain_max_phases` of them that follow one another
    are launched as ONE kernel, in which each starts fetching its weights while the one before it is
    still being finished.  Every other op of this module launches what is pending before it runs, so
    a caller that only uses these ops sees no difference; code that reads a product's output by
    other means (a torch op) calls `flush_gemm_chain()` first.  Nothing happens when `enabled` is
    false, and chains do not nest."""

    def __init__(self, device: torch.device, enabled: bool = True) -> None:
        self.device, self.enabled = device, bool(enabled)

    def __enter__(self):
        global _chain_open, _chain_counted
        self.mine = self.enabled and not _chain_open
        if self.mine:
            fn = library().ts_gemm_chain_begin
            fn.argtypes = [_c_void_p]
            fn.restype = None
            fn(_chain_sync_words(self.device).data_ptr())
            _chain_open = True
            _chain_counted = 0
        return self

    def __exit__(self, *exc):
        global _chain_open
        if self.mine:
            try:
                flush_gemm_chain(end=True)
            finally:
                _chain_open = False
                _chain_keep.clear()
        return False


def flush_gemm_chain(end: bool = False) -> None:
    """Launches the products that wait in the chain (nothing, if no chain is open)."""
    global launch_count, _chain_counted
    if not _chain_open:
        return
    lib = library()
    status = (lib.ts_gemm_chain_end if end else lib.ts_gemm_chain_flush)()
    launched = lib.ts_gemm_chain_launches()
    launch_count += launched - _chain_counted
    _chain_counted = launched
    _chain_keep.clear()
    if status != 0:
        raise KernelError(f"chained products: CUDA error {status} at launch")


def _check_product(name: str, status: int, *tensors) -> None:
    """_check for a product that may have joined a chain instead of being launched."""
    global launch_count, _chain_counted
    if not _chain_open:
        _check(name, status)
        return
    _chain_keep.append(tensors)
    launched = library().ts_gemm_chain_launches()  # a full list, or another row count, launched what was pending
    launch_count += launched - _chain_counted
    _chain_counted = launched
    if status != 0:
        _check(name, status)


def embed_gather(hidden: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """hidden[t] = table[ids[t]] widened to float32.  hidden [T,H] f32, table [V,H], ids [T] i32."""
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    _cuda_contig("table", table)
    _cuda_contig("ids", ids, torch.int32)
    T, H = hidden.shape
    V = table.shape[0]
    if table.shape[1] != H or ids.numel() < T:
        raise KernelError(f"embed_gather: shapes disagree: hidden {tuple(hidden.shape)}, table {tuple(table.shape)}, ids {tuple(ids.shape)}")
    _check("embed_gather", _fn("ts_embed_gather")(
        hidden.data_ptr(), table.data_ptr(), _act_code("table", table), ids.data_ptr(), T, H, V, _stream()))


def feed_tokens(ids: torch.Tensor, source: torch.Tensor, lanes: torch.Tensor, rows: torch.Tensor, n: int) -> None:
    """ids[lanes[i]] = source[rows[i]] for i < n (all int32, on the device): token ids that an
    earlier kernel produced go into a step's inputs without passing through the host."""
    flush_gemm_chain()
    for name, t in (("ids", ids), ("source", source), ("lanes", lanes), ("rows", rows)):
        _cuda_contig(name, t, torch.int32)
    if n > lanes.numel() or n > rows.numel():
        raise KernelError(f"feed_tokens: {n} lanes, but the index arrays hold {lanes.numel()} and {rows.numel()}")
    _check("feed_tokens", _fn("ts_feed_tokens")(ids.data_ptr(), source.data_ptr(), lanes.data_ptr(), rows.data_ptr(), int(n), _stream()))


def add_rmsnorm(
    hidden: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    row_index: Optional[torch.Tensor] = None,
) -> None:
    """hidden += delta (float32, in place) and out = RMSNorm(hidden) * weight.

    hidden [T,H] f32; delta [T,H] of out's dtype or None; weight [H] f32; out [rows,H].
    With `row_index` ([rows] i32) only those rows are normed and hidden is left as it is.
    """
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("out", out)
    H = hidden.shape[-1]
    rows = out.shape[0]
    if out.shape[-1] != H or weight.numel() != H:
        raise KernelError(f"add_rmsnorm: widths disagree: hidden {tuple(hidden.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if delta is not None:
        _cuda_contig("delta", delta, out.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("add_rmsnorm: delta must have hidden's shape")
    if row_index is not None:
        _cuda_contig("row_index", row_index, torch.int32)
        if row_index.numel() < rows:
            raise KernelError("add_rmsnorm: row_index is shorter than out")
    elif rows != hidden.shape[0]:
        raise KernelError("add_rmsnorm: out must have hidden's rows when no row_index is given")
    _check("add_rmsnorm", _fn("ts_add_rmsnorm")(
        hidden.data_ptr(), _ptr(delta), _act_code("out", out), weight.data_ptr(), out.data_ptr(),
        _ptr(row_index), rows, H, float(eps), _stream()))


def residual_add(hidden: torch.Tensor, delta: torch.Tensor) -> None:
    """hidden += delta in float32.  hidden [T,H] f32, delta [T,H] f32 or bf16."""
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    _cuda_contig("delta", delta)
    if delta.shape != hidden.shape:
        raise KernelError("residual_add: shapes disagree")
    _check("residual_add", _fn("ts_residual_add")(
        hidden.data_ptr(), delta.data_ptr(), _act_code("delta", delta), hidden.numel(), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[t,i] = silu(gate[t,i]) * up[t,i].  gate_up [T,2I], out [T,I].  block 0: gate i at column
    i, up at I + i; block 64: blocks of 128 columns, 64 gates and then their 64 ups."""
    flush_gemm_chain()
    _cuda_contig("gate_up", gate_up)
    _cuda_contig("out", out, gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    if block not in (0, 64) or (block and I % 64):
        raise KernelError(f"swiglu: block must be 0 or 64 (and then divide the width), got {block} for width {I}")
    _check("swiglu", _fn("ts_swiglu")(gate_up.data_ptr(), out.data_ptr(), _act_code("out", out), T, I, int(block), _stream()))


QK_ROPE_MAX_HEAD_DIM = 512


def qk_norm_rope_store(
    qkv: torch.Tensor,
    q_out: torch.Tensor,
    k_dst: Optional[torch.Tensor],
    v_dst: Optional[torch.Tensor],
    slot_mapping: Optional[torch.Tensor],
    positions: torch.Tensor,
    q_norm_weight: Optional[torch.Tensor],
    k_norm_weight: Optional[torch.Tensor],
    eps: float,
    inv_freq: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
) -> None:
    """Per-head q/k RMSNorm, rotary encoding, and the key/value store.

    qkv [T,(nq+2nkv)*d]; q_out [T,nq*d]; k_dst/v_dst: the cache pools [slots,nkv,d] (with
    `slot_mapping` [T] i32, -1 = skip) or dense [T,nkv,d] buffers (slot_mapping None).
    Norm weights [d] f32 or None (no norm); inv_freq [rot/2] f32 or None (no rotation);
    a rotation narrower than d leaves the upper dims as they are.
    """
    flush_gemm_chain()
    _cuda_contig("qkv", qkv)
    _cuda_contig("q_out", q_out, qkv.dtype)
    _cuda_contig("positions", positions, torch.int32)
    T = qkv.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if d > QK_ROPE_MAX_HEAD_DIM or d % 2:
        raise KernelError(f"qk_norm_rope_store: head_dim must be even and <= {QK_ROPE_MAX_HEAD_DIM}, got {d}")
    if qkv.shape[1] != (nq + 2 * nkv) * d or q_out.numel() != T * nq * d:
        raise KernelError(f"qk_norm_rope_store: qkv {tuple(qkv.shape)} / q_out {tuple(q_out.shape)} do not match heads {nq}+2*{nkv} of {d}")
    if nkv > 0:
        for name, c in (("k_dst", k_dst), ("v_dst", v_dst)):
            if c is None:
                raise KernelError(f"qk_norm_rope_store: {name} is required")
            _cuda_contig(name, c, qkv.dtype)
            if c.shape[-1] != d or c.shape[-2] != nkv:
                raise KernelError(f"qk_norm_rope_store: {name} must end in [{nkv},{d}], got {tuple(c.shape)}")
        if slot_mapping is None and (k_dst.numel() < T * nkv * d or v_dst.numel() < T * nkv * d):
            raise KernelError("qk_norm_rope_store: dense k/v buffers are too small")
    if slot_mapping is not None:
        _cuda_contig("slot_mapping", slot_mapping, torch.int32)
        if slot_mapping.numel() < T:
            raise KernelError("qk_norm_rope_store: slot_mapping is shorter than the batch")
    if positions.numel() < T:
        raise KernelError("qk_norm_rope_store: positions is shorter than the batch")
    for name, w in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight)):
        if w is not None:
            _cuda_contig(name, w, torch.float32)
            if w.numel() != d:
                raise KernelError(f"qk_norm_rope_store: {name} must have {d} entries")
    rot = 0
    if inv_freq is not None:
        _cuda_contig("inv_freq", inv_freq, torch.float32)
        rot = 2 * inv_freq.numel()
        if rot > d or rot <= 0:
            raise KernelError(f"qk_norm_rope_store: rotary width {rot} does not fit head_dim {d}")
    _check("qk_norm_rope_store", _fn("ts_qk_norm_rope_store")(
        qkv.data_ptr(), _act_code("qkv", qkv), q_out.data_ptr(), _ptr(k_dst), _ptr(v_dst),
        _ptr(slot_mapping), positions.data_ptr(), _ptr(q_norm_weight), _ptr(k_norm_weight),
        float(eps), _ptr(inv_freq), rot, T, nq, nkv, d, _stream()))


ATTENTION_SIMPLE_MAX_HEAD_DIM = 512


def attention_paged_simple(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    positions: torch.Tensor,
    seq_index: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int = 0,
) -> None:
    """Causal attention over the paged cache on CUDA cores (float32 or bfloat16).

    q/out [T,nq*d]; caches [pages,page,nkv,d]; positions, seq_index [T] i32;
    block_table [B,max_blocks] i32.  window > 0: a query sees its last `window` keys.
    """
    flush_gemm_chain()
    _cuda_contig("q", q)
    _cuda_contig("k_cache", k_cache, q.dtype)
    _cuda_contig("v_cache", v_cache, q.dtype)
    _cuda_contig("out", out, q.dtype)
    _cuda_contig("positions", positions, torch.int32)
    _cuda_contig("seq_index", seq_index, torch.int32)
    _cuda_contig("block_table", block_table, torch.int32)
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if d > ATTENTION_SIMPLE_MAX_HEAD_DIM:
        raise KernelError(f"attention_paged_simple: head_dim must be <= {ATTENTION_SIMPLE_MAX_HEAD_DIM}, got {d}")
    if nq % nkv:
        raise KernelError(f"attention: {nq} query heads are no multiple of {nkv} key/value heads")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention: q/out do not match [T, heads*head_dim]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or positions.numel() < T or seq_index.numel() < T:
        raise KernelError("attention: block_table must be [B,max_blocks]; positions and seq_index need T entries")
    _check("attention_paged_simple", _fn("ts_attention_paged_simple")(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _act_code("q", q), out.data_ptr(),
        positions.data_ptr(), seq_index.data_ptr(), block_table.data_ptr(), block_table.shape[1],
        page_size, T, nq, nkv, d, float(scale), int(window), _stream()))


def sample(
    logits: torch.Tensor,
    temperature: torch.Tensor,
    keys: Optional[torch.Tensor],
    out: torch.Tensor,
) -> None:
    """One token per row of float32 logits [R,V]: argmax where temperature is 0, else the
    exponential race keyed by keys[r] (int64, the noise stream of that row).  out [R] i32."""
    flush_gemm_chain()
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a float32 CUDA matrix with unit inner stride")
    _cuda_contig("temperature", temperature, torch.float32)
    _cuda_contig("out", out, torch.int32)
    R, V = logits.shape
    if keys is not None:
        _cuda_contig("keys", keys, torch.int64)
        if keys.numel() < R:
            raise KernelError("sample: keys is shorter than the batch")
    if temperature.numel() < R or out.numel() < R:
        raise KernelError("sample: temperature/out are shorter than the batch")
    # stage 1 leaves one (value, index) pair per 2048-entry chunk of each row for stage 2
    scratch = torch.empty(R * (-(-V // 2048)) * 2, dtype=torch.int32, device=logits.device)
    _check("sample", _fn("ts_sample")(
        logits.data_ptr(), V, logits.stride(0), temperature.data_ptr(), _ptr(keys), out.data_ptr(), R,
        scratch.data_ptr(), _stream()))
    global launch_count
    launch_count += 1  # two kernels per call


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true float32 (FFMA)."""
    flush_gemm_chain()
    for name, t in (("a", a), ("w", w), ("out", out)):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"sgemm_nt: {name} must be a float32 CUDA matrix with unit inner stride")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"sgemm_nt: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check("sgemm_nt", _fn("ts_sgemm_nt")(
        a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), w.stride(0), out.stride(0), _stream()))


# ---------------------------------------------------------------------------
# tensor-core attention (one library per head size)

# Decode steps with 2..8 key splits: the splits of a (sequence, KV head) pair form a thread-block
# cluster and merge through its shared memory (TS_ATTENTION_CLUSTER=0: scratch and a second kernel).
ATTENTION_CLUSTER_MERGE = _os.environ.get("TS_ATTENTION_CLUSTER", "1") != "0"
# Decode steps fetch keys and values with the copy engine (TMA) where the sizes allow it: head sizes
# that are multiples of 64, pages of at least 8 slots that divide 64 or are multiples of it
# (TS_ATTENTION_TMA=0: 16-byte asynchronous copies by the threads, which take every size).
ATTENTION_DECODE_TMA = _os.environ.get("TS_ATTENTION_TMA", "1") != "0"
_attention_error: Optional[torch.Tensor] = None


def _pinned_word() -> torch.Tensor:
    """One zeroed int32 in pinned host memory that kernels may write and the host reads without a
    copy.  Made outside inference mode, so that the host may clear it from anywhere."""
    with torch.inference_mode(False):
        return torch.zeros(1, dtype=torch.int32).pin_memory()


def _word_is_set(word: torch.Tensor) -> bool:
    """Reads and clears an error word through its numpy view (plain memory, no tensor dispatch)."""
    view = word.numpy()
    if int(view[0]) == 0:
        return False
    view[0] = 0
    return True


def _attention_error_word() -> torch.Tensor:
    """One int in pinned host memory that the decode attention sets when a bounded wait gave up."""
    global _attention_error
    if _attention_error is None:
        _attention_error = _pinned_word()
    return _attention_error


ATTENTION_MMA_MAX_HEAD_DIM = 256
ATTENTION_MMA_MAX_SPLITS = 64
_attention_mma: dict[int, tuple] = {}


def attention_mma_supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= ATTENTION_MMA_MAX_HEAD_DIM


def _attention_mma_fns(head_dim: int):
    fns = _attention_mma.get(head_dim)
    if fns is None:
        if not attention_mma_supported(head_dim):
            raise KernelError(
                f"attention_paged_mma: head_dim must be a multiple of 16 between 16 and {ATTENTION_MMA_MAX_HEAD_DIM}, got {head_dim}")
        lib = _build.load_variant("attention_mma", {"TS_HEAD_DIM": head_dim})
        run = lib.ts_attention_paged_mma_fused
        run.argtypes = [_c_void_p] * 9 + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_int, _c_void_p, _c_void_p]
        run.restype = _c_int
        scratch = lib.ts_attention_mma_scratch_floats
        scratch.argtypes = [_c_ll, _c_int]
        scratch.restype = _c_ll
        if lib.ts_attention_mma_head_dim() != head_dim:
            raise KernelError("attention_paged_mma: the loaded library was built for another head size")
        lib.ts_attention_mma_set_cluster_merge.argtypes = [_c_int]
        lib.ts_attention_mma_set_cluster_merge(1 if ATTENTION_CLUSTER_MERGE else 0)
        lib.ts_attention_mma_set_decode_tma.argtypes = [_c_int]
        lib.ts_attention_mma_set_decode_tma(1 if ATTENTION_DECODE_TMA else 0)
        lib.ts_attention_mma_set_error_word.argtypes = [_c_void_p]
        lib.ts_attention_mma_set_error_word(_attention_error_word().data_ptr())
        lib.ts_attention_decode_flat.argtypes = [_c_void_p] * 9 + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void_p]
        lib.ts_attention_decode_flat.restype = _c_int
        lib.ts_attention_decode_flat_ctas.restype = _c_int
        lib.ts_attention_decode_flat_scratch_floats.argtypes = [_c_int, _c_int]
        lib.ts_attention_decode_flat_scratch_floats.restype = _c_ll
        lib.ts_attention_mma_decode_slots.restype = _c_ll
        lib.ts_attention_mma_decode_rows.restype = _c_int
        lib.ts_attention_mma_last_launches.restype = _c_int
        _attention_flat[head_dim] = lib
        fns = (run, scratch)
        _attention_mma[head_dim] = fns
    return fns


_decode_slot_counts: dict[int, int] = {}


def _decode_slots(head_dim: int) -> int:
    """CTAs of the decode attention kernel that run at once on this device, as the library's
    occupancy query for the real kernel says."""
    n = _decode_slot_counts.get(head_dim)
    if n is None:
        _attention_mma_fns(head_dim)
        n = _decode_slot_counts[head_dim] = max(1, int(_attention_flat[head_dim].ts_attention_mma_decode_slots()))
    return n


def attention_decode_rows(head_dim: int) -> int:
    """The most query rows (tokens of the step x query heads per key/value head) of one sequence
    that the decode kernels take; steps with more go to the prompt kernels."""
    _attention_mma_fns(head_dim)
    return int(_attention_flat[head_dim].ts_attention_mma_decode_rows())


# The context length the split count of a decode step is planned for when the step may serve any
# length up to the model's (a captured graph does): long enough that a few thousand keys are spread
# over all SMs, short enough that a sequence of a few hundred keys is not cut into slivers
# (TS_DECODE_PLAN_CONTEXT overrides it for measurements).
ATTENTION_DECODE_PLAN_CONTEXT = int(_os.environ.get("TS_DECODE_PLAN_CONTEXT", "2048"))


def attention_decode_plan_context(max_context: int, window: int = 0) -> int:
    """The context length to plan a decode step's key splits for: the longest the step can meet,
    capped by the window (plus one key block) or by ATTENTION_DECODE_PLAN_CONTEXT."""
    cap = window + 64 if window > 0 else ATTENTION_DECODE_PLAN_CONTEXT
    return max(1, min(max_context, cap))


def attention_decode_splits(num_seqs: int, num_kv_heads: int, max_context: int, head_dim: int = 128) -> int:
    """How many CTAs share the keys of one sequence in a decode step.

    Each (sequence, KV head) pair is one unit of work that `splits` CTAs divide evenly.  The
    GPU runs `slots` CTAs at a time (shared memory allows a few per SM, fewer for large
    heads); the step takes ceil(pairs * splits / slots) waves, each as long as one CTA's
    share, so the count is chosen to fill whole waves: one wave for small batches, and for
    batches with more pairs than slots a count that makes the last wave nearly full.
    """
    slots = _decode_slots(head_dim)
    pairs = max(1, num_seqs * num_kv_heads)
    blocks = max(1, -(-max_context // 64))
    if _os.environ.get("TS_DECODE_SPLITS"):
        return max(1, min(int(_os.environ["TS_DECODE_SPLITS"]), blocks, ATTENTION_MMA_MAX_SPLITS))
    best, best_cost = 1, None
    for s in range(1, min(blocks, 16) + 1):
        waves = -(-pairs * s // slots)
        # per CTA: start and merge (about 3 us) + 2.5 us per 64-key block; merging the splits costs
        # little inside a thread-block cluster (up to 8 CTAs, all running at once), more through
        # scratch and a kernel of its own
        in_cluster = ATTENTION_CLUSTER_MERGE and s <= 8 and pairs * s <= slots
        merge = 0.0 if s == 1 else (0.8 if in_cluster else 1.5 + 0.15 * s)
        cost = waves * (3.0 + 2.5 * -(-blocks // s)) + merge
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def attention_decode_plan(num_seqs: int, num_kv_heads: int, max_context: int, head_dim: int = 128) -> tuple[int, int]:
    """(splits, keys_per_split) for fixed-size key chunks: every (sequence, KV head) pair is cut
    into chunks of `keys_per_split` keys, one CTA each; `splits` chunks cover `max_context`, and
    sequences shorter than that use fewer of their CTAs.  For batches whose longest context is
    known when the step is launched."""
    pairs = max(1, num_seqs * num_kv_heads)
    chunk = 64 if pairs <= 16 else (128 if pairs <= 64 else 256)
    splits = -(-max(1, max_context) // chunk)
    while splits > ATTENTION_MMA_MAX_SPLITS:
        chunk *= 2
        splits = -(-max_context // chunk)
    if splits <= 1:
        return 1, 0
    return splits, chunk


def attention_paged_mma(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    context_lens: torch.Tensor,
    block_table: torch.Tensor,
    seq_index: torch.Tensor,
    page_size: int,
    num_seqs: int,
    max_seqlen_q: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int = 0,
    splits: int = 1,
    scratch: Optional[torch.Tensor] = None,
    keys_per_split: int = 0,
    fuse_merge: bool = True,
) -> None:
    """Causal attention over the paged cache on tensor cores (bfloat16).

    q/out [T,nq*d]; caches [pages,page,nkv,d]; cu_seqlens_q [B+1], context_lens [B],
    seq_index [T] i32; block_table [B,max_blocks] i32.  The tokens of a sequence are
    consecutive and end at context_lens[b] - 1.  splits > 1 spreads the keys of a
    sequence over several CTAs and needs `scratch` (float32, see attention_scratch_floats);
    keys_per_split > 0 (a multiple of 64) gives split s the keys [s * keys_per_split, ...),
    0 divides each sequence's keys evenly.  In decode steps the last CTA of each (sequence, KV
    head) pair merges the pair's splits itself (`fuse_merge`); otherwise a second kernel does.
    """
    flush_gemm_chain()
    run, _ = _attention_mma_fns(head_dim)
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _cuda_contig(name, t, torch.bfloat16)
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("context_lens", context_lens), ("block_table", block_table), ("seq_index", seq_index)):
        _cuda_contig(name, t, torch.int32)
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if nq % nkv:
        raise KernelError(f"attention: {nq} query heads are no multiple of {nkv} key/value heads")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention: q/out do not match [T, heads*head_dim]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or block_table.shape[0] < num_seqs:
        raise KernelError("attention: block_table must be [B,max_blocks]")
    if cu_seqlens_q.numel() < num_seqs + 1 or context_lens.numel() < num_seqs or seq_index.numel() < T:
        raise KernelError("attention: cu_seqlens_q/context_lens/seq_index are shorter than the batch")
    if keys_per_split < 0 or keys_per_split % 64:
        raise KernelError(f"attention: keys_per_split must be a multiple of 64, got {keys_per_split}")
    if not (1 <= splits <= ATTENTION_MMA_MAX_SPLITS):
        raise KernelError(f"attention: splits must be 1..{ATTENTION_MMA_MAX_SPLITS}, got {splits}")
    if splits > 1:
        need = attention_scratch_floats(T * nq, splits, d)
        if scratch is None or scratch.dtype != torch.float32 or not scratch.is_cuda or scratch.numel() < need:
            raise KernelError(f"attention: splits={splits} needs {need} float32 of scratch")
    counters = None
    if fuse_merge and _FUSE_ATTENTION_MERGE and splits > 1 and max_seqlen_q * (nq // nkv) <= attention_decode_rows(d) and num_seqs * nkv <= _GEMM_MAX_TILES:
        counters = _attention_counters(q.device).data_ptr()
    _check("attention_paged_mma", run(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _ptr(scratch),
        cu_seqlens_q.data_ptr(), context_lens.data_ptr(), block_table.data_ptr(), seq_index.data_ptr(),
        block_table.shape[1], page_size, T, num_seqs, max_seqlen_q, nq, nkv, float(scale), int(window), int(splits),
        int(keys_per_split), counters, _stream()))
    if splits > 1:
        global launch_count
        launch_count += _attention_flat[d].ts_attention_mma_last_launches() - 1  # the combine kernel, if one ran


# Decode steps whose (sequence, KV head) pairs times key splits do not all run at once go to the
# kernel that gives every CTA an even share of all key blocks instead (TS_ATTENTION_FLAT=0: never).
ATTENTION_DECODE_FLAT = _os.environ.get("TS_ATTENTION_FLAT", "1") != "0"
ATTENTION_FLAT_MAX_SEQS = 512
ATTENTION_FLAT_MAX_ROWS = 16
_attention_flat: dict[int, ctypes.CDLL] = {}
_flat_ctas: dict[int, int] = {}


def attention_decode_flat_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, num_seqs: int, max_seqlen_q: int) -> bool:
    """Whether the even-share decode kernel takes these sizes: head sizes that are multiples of 64,
    pages the copy engine can fetch (8 or more slots; 64 a multiple of the page or the page of 64),
    at most 16 rows (tokens x heads of a group) per sequence and KV head, at most 512 sequences."""
    return (head_dim % 64 == 0 and attention_mma_supported(head_dim) and num_kv_heads > 0 and num_heads % num_kv_heads == 0
            and page_size >= 8 and (64 % page_size == 0 or page_size % 64 == 0)
            and max_seqlen_q * (num_heads // num_kv_heads) <= ATTENTION_FLAT_MAX_ROWS and 0 < num_seqs <= ATTENTION_FLAT_MAX_SEQS
            and (num_kv_heads * head_dim * 2) % 16 == 0)


def attention_decode_prefers_flat(num_seqs: int, num_kv_heads: int, splits: int, head_dim: int) -> bool:
    """Whether a decode step of this many sequences is better served by the even-share kernel:
    when the CTAs of the split kernel would queue (measured at 8 KV heads of 128: equal at 32
    sequences, 19 % faster at 64, 10 % at 128; with fewer sequences the split kernel, whose
    splits merge inside a cluster, is faster)."""
    return ATTENTION_DECODE_FLAT and num_seqs * num_kv_heads * splits > _decode_slots(head_dim)


def attention_decode_flat_ctas(head_dim: int) -> int:
    """CTAs of the even-share decode kernel that the GPU runs at once: its grid."""
    n = _flat_ctas.get(head_dim)
    if n is None:
        _attention_mma_fns(head_dim)
        n = int(_attention_flat[head_dim].ts_attention_decode_flat_ctas())
        _flat_ctas[head_dim] = n
    return n


def attention_decode_flat(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    context_lens: torch.Tensor,
    block_table: torch.Tensor,
    seq_index: torch.Tensor,
    page_size: int,
    num_seqs: int,
    max_seqlen_q: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int = 0,
    ctas: int = 0,
) -> None:
    """Decode attention over the paged cache with an even share of key blocks per CTA (bfloat16).

    Arguments as attention_paged_mma.  The key blocks (64 keys) of all (sequence, KV head) pairs
    form one list that the CTAs of a fixed grid divide evenly on the device, whatever the lengths
    are; pairs that several CTAs share are merged by a second kernel.  `ctas` (0: as many as run
    at once) sets the grid."""
    flush_gemm_chain()
    _attention_mma_fns(head_dim)
    lib = _attention_flat[head_dim]
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _cuda_contig(name, t, torch.bfloat16)
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("context_lens", context_lens), ("block_table", block_table), ("seq_index", seq_index)):
        _cuda_contig(name, t, torch.int32)
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if not attention_decode_flat_supported(nq, nkv, d, page_size, num_seqs, max_seqlen_q):
        raise KernelError(
            f"attention_decode_flat: takes head sizes that are multiples of 64, pages of 8 or more slots that divide 64 or are multiples of it, "
            f"at most {ATTENTION_FLAT_MAX_ROWS} rows per sequence and KV head and at most {ATTENTION_FLAT_MAX_SEQS} sequences; got "
            f"heads {nq}/{nkv} of {d}, page {page_size}, {num_seqs} sequences of up to {max_seqlen_q} tokens")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention_decode_flat: q/out do not match [T, heads*head_dim]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_decode_flat: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or block_table.shape[0] < num_seqs:
        raise KernelError("attention_decode_flat: block_table must be [B,max_blocks]")
    if cu_seqlens_q.numel() < num_seqs + 1 or context_lens.numel() < num_seqs or seq_index.numel() < T:
        raise KernelError("attention_decode_flat: cu_seqlens_q/context_lens/seq_index are shorter than the batch")
    most = attention_decode_flat_ctas(d)
    ctas = most if ctas <= 0 else min(int(ctas), most)
    scratch = torch.empty(int(lib.ts_attention_decode_flat_scratch_floats(num_seqs, ctas)), device=q.device, dtype=torch.float32)
    _check("attention_decode_flat", lib.ts_attention_decode_flat(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), scratch.data_ptr(),
        cu_seqlens_q.data_ptr(), context_lens.data_ptr(), block_table.data_ptr(), seq_index.data_ptr(),
        block_table.shape[1], page_size, T, num_seqs, max_seqlen_q, nq, nkv, float(scale), int(window), ctas, _stream()))
    global launch_count
    launch_count += 1  # the combine kernel


_FUSE_ATTENTION_MERGE = _os.environ.get("TS_FUSE_ATTENTION_MERGE", "0") != "0"  # measured: the separate merge kernel is a little faster
_attention_counter_tensors: dict[tuple[int, int], torch.Tensor] = {}


def _attention_counters(device: torch.device) -> torch.Tensor:
    """Per (device, stream): ticket counters of the decode attention's key splits (zero between launches)."""
    key = (device.index or 0, _stream())
    t = _attention_counter_tensors.get(key)
    if t is None:
        t = _attention_counter_tensors[key] = torch.zeros(_GEMM_MAX_TILES, dtype=torch.int32, device=device)
    return t


def attention_scratch_floats(rows: int, splits: int, head_dim: int) -> int:
    return rows * splits * (head_dim + 2) if splits > 1 else 0


# ---------------------------------------------------------------------------
# prompt attention on tcgen05 tensor cores (head size 128)

ATTENTION_TCGEN05_HEAD_DIM = 128
_attention_tcgen05 = None
_USE_ATTENTION_TCGEN05 = _os.environ.get("TS_ATTENTION_TCGEN05", "1") != "0"


def _attention_tcgen05_fns():
    global _attention_tcgen05
    if _attention_tcgen05 is None:
        lib = _build.load_variant("attention_tcgen05", {"TS_HEAD_DIM": ATTENTION_TCGEN05_HEAD_DIM})
        run = lib.ts_attention_prefill_tcgen05
        run.argtypes = [_c_void_p] * 7 + [_c_int, _c_int, _c_ll] + [_c_int] * 5 + [_c_float, _c_int, _c_int, _c_void_p, _c_void_p]
        run.restype = _c_int
        ok = lib.ts_attention_tcgen05_supported
        ok.argtypes = [_c_int, _c_int, _c_int]
        ok.restype = _c_int
        _attention_tcgen05 = (run, ok)
    return _attention_tcgen05


def attention_tcgen05_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes these sizes: head size 128, at most 128
    query heads per key/value head (a tile of 128 rows holds whole tokens: 128 // group of them), a
    page size of at least 8 that divides 64 or is a multiple of 128."""
    if not _USE_ATTENTION_TCGEN05 or head_dim != ATTENTION_TCGEN05_HEAD_DIM:
        return False
    if num_kv_heads <= 0 or num_heads % num_kv_heads or num_heads // num_kv_heads > 128:
        return False
    return page_size >= 8 and (64 % page_size == 0 or page_size % 128 == 0)


def attention_prefill_tcgen05(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    context_lens: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    num_seqs: int,
    max_seqlen_q: int,
    num_heads: int,
    num_kv_heads: int,
    scale: float,
    window: int = 0,
    mode: int = 0,
) -> None:
    """Causal attention of prompt portions over the paged cache, tcgen05 tensor cores, head size 128.

    Same arguments and meaning as attention_paged_mma (without seq_index, which it does not need).
    `mode`: 1 one tile of 128 rows per CTA, 2 two tiles per CTA with the roles in warps of
    their own, 0 chooses by the longest portion.
    """
    flush_gemm_chain()
    run, ok = _attention_tcgen05_fns()
    d = ATTENTION_TCGEN05_HEAD_DIM
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _cuda_contig(name, t, torch.bfloat16)
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("context_lens", context_lens), ("block_table", block_table)):
        _cuda_contig(name, t, torch.int32)
    T = q.shape[0]
    nq, nkv = num_heads, num_kv_heads
    if not ok(nq, nkv, page_size):
        raise KernelError(
            f"attention_prefill_tcgen05: needs at most 128 query heads per key/value head and a page size of at least 8 that divides 64 or is a multiple of 128; "
            f"got {nq} query heads, {nkv} key/value heads, pages of {page_size}")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention_prefill_tcgen05: q/out do not match [T, heads*128]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_prefill_tcgen05: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or block_table.shape[0] < num_seqs:
        raise KernelError("attention_prefill_tcgen05: block_table must be [B,max_blocks]")
    if cu_seqlens_q.numel() < num_seqs + 1 or context_lens.numel() < num_seqs:
        raise KernelError("attention_prefill_tcgen05: cu_seqlens_q/context_lens are shorter than the batch")
    _, error = _gemm_workspace(q.device)
    _check("attention_prefill_tcgen05", run(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        cu_seqlens_q.data_ptr(), context_lens.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, k_cache.shape[0] * page_size, T, num_seqs, max_seqlen_q, nq, nkv,
        float(scale), int(window), int(mode), error.data_ptr(), _stream()))


# ---------------------------------------------------------------------------
# skinny GEMM on tcgen05 tensor cores (decode steps)

GEMM_SKINNY_MAX_ROWS = 128
_SIGNATURES["ts_gemm_skinny_bf16"] = [
    _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_int,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p,
]
# How much of the next GEMM's weights a GEMM asks into L2 while its own last tiles are finished.
# Measured on the decode step at batch 8 (ms per step, the weights themselves passing through the
# L2 as "evict first"): none 3.87, 8 MB 3.83, 16 MB 3.80, 24 MB 3.82, 32 MB 3.84, 48 MB 3.86,
# 96 MB 3.94 (the requests then compete with the kernel's own tail).  TS_GEMM_PREFETCH_MB
# overrides it for measurements.
GEMM_PREFETCH_BYTES = int(_os.environ.get("TS_GEMM_PREFETCH_MB", "16")) << 20
_gemm_workspaces: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}
_CHAIN_SYNC_WORDS = 512  # at least ts_gemm_chain_sync_words(), on a 128-byte boundary behind the tickets


def _gemm_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Per (device, stream): the ticket counters of the K-split tiles (zero between launches)
    and the error word, which lives in pinned host memory so the host can look at it without
    a copy."""
    key = (device.index or 0, _stream())
    ws = _gemm_workspaces.get(key)
    if ws is None:
        counters = torch.zeros(_GEMM_MAX_TILES + _CHAIN_SYNC_WORDS, dtype=torch.int32, device=device)  # tickets, then the chain's barrier words
        error = _pinned_word()
        ws = _gemm_workspaces[key] = (counters, error)
    return ws


_gemm_partials: dict[tuple[int, int], torch.Tensor] = {}
_gemm_partials_outgrown: list[torch.Tensor] = []
_gemm_scratch_need: dict[tuple[int, int, int], int] = {}


def _gemm_partial(device: torch.device, M: int, N: int, K: int) -> torch.Tensor:
    """Per (device, stream): the float32 scratch in which CTAs that share a tile meet.  One buffer
    serves every launch on the stream (it only grows): a GEMM stores nothing before the kernels
    ahead of it are done, so two launches never use it at once."""
    need = _gemm_scratch_need.get((M, N, K))
    if need is None:
        scratch_floats = library().ts_gemm_skinny_scratch_floats
        scratch_floats.restype = _c_ll
        need = _gemm_scratch_need[(M, N, K)] = max(4, int(scratch_floats(M, N, K)))
    key = (device.index or 0, _stream())
    buf = _gemm_partials.get(key)
    if buf is None or buf.numel() < need:
        if buf is not None:
            _gemm_partials_outgrown.append(buf)  # a captured graph may still name it: never handed back
        buf = _gemm_partials[key] = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=device)
    return buf


class _MatrixFacts:
    """What the GEMM wrappers ask of a weight matrix again and again, looked up once and kept on the
    tensor object (a weight does not change its place or shape while it lives)."""

    __slots__ = ("ok", "ptr", "rows", "cols", "ld", "nbytes")

    def __init__(self, w: torch.Tensor) -> None:
        self.ptr = w.data_ptr()
        self.rows, self.cols = (int(w.shape[0]), int(w.shape[1])) if w.dim() == 2 else (0, 0)
        self.ld = int(w.stride(0)) if w.dim() == 2 else 0
        self.nbytes = w.numel() * w.element_size()
        self.ok = bool(
            w.dim() == 2 and w.is_cuda and w.dtype == torch.bfloat16 and self.cols % 8 == 0 and w.stride(1) == 1
            and self.ld % 8 == 0 and self.ptr % 16 == 0 and -(-self.rows // 128) <= _GEMM_MAX_TILES)


def _facts(w: torch.Tensor) -> _MatrixFacts:
    f = getattr(w, "_ts_facts", None)
    if f is None or f.ptr != w.data_ptr():
        f = _MatrixFacts(w)
        try:
            w._ts_facts = f
        except (AttributeError, RuntimeError):  # an object that takes no attributes: look it up every time
            pass
    return f


def matrix_streams_through_own_gemm(w: Optional[torch.Tensor]) -> bool:
    """Whether `w` ([out, in], bfloat16, on the device, rows on 16-byte boundaries, in % 8 == 0) is a
    weight the engine's own few-row GEMM takes."""
    return w is not None and _facts(w).ok


def gemm_skinny_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    M, K = x.shape
    return (
        _facts(w).ok and x.dtype == torch.bfloat16 and 0 < M <= GEMM_SKINNY_MAX_ROWS and K % 8 == 0
        and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
    )


_gemm_scratch_ptrs: dict[tuple[int, int], tuple[int, int, int, int]] = {}


def _gemm_scratch(device: torch.device, M: int, N: int, K: int) -> tuple[int, int, int, int]:
    """(partial sums, ticket counters, error word, stream) as plain addresses for one launch on the
    current stream: the buffers of _gemm_partial and _gemm_workspace, looked up with one query of
    the stream."""
    stream = _stream()
    key = (device.index or 0, stream)
    need = _gemm_scratch_need.get((M, N, K))
    got = _gemm_scratch_ptrs.get(key)
    if need is None or got is None or got[3] < need:
        partial = _gemm_partial(device, M, N, K)
        counters, error = _gemm_workspace(device)
        got = _gemm_scratch_ptrs[key] = (partial.data_ptr(), counters.data_ptr(), error.data_ptr(), partial.numel())
    return got[0], got[1], got[2], stream


def gemm_skinny_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, prefetch: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = x[M,K] @ w[N,K]^T for M <= 128 on the tcgen05 tensor cores.

    x, w bfloat16 with unit inner stride and rows that start on 16-byte boundaries; out
    bfloat16 or float32.  The work is spread evenly over all SMs; tiles that two CTAs share
    meet in a float32 scratch that this wrapper allocates.  `prefetch`: the weights the next
    product will read; the kernel asks for their start to be brought into L2 while it finishes.
    """
    if not (x.is_cuda and w.is_cuda and out.is_cuda):
        raise KernelError("gemm_skinny_bf16: CUDA tensors only (there is no CPU path)")
    if not gemm_skinny_supported(x, w):
        raise KernelError(
            f"gemm_skinny_bf16: needs bfloat16, at most {GEMM_SKINNY_MAX_ROWS} rows, K a multiple of 8 and 16-byte "
            f"aligned rows; got x {tuple(x.shape)} {x.dtype} strides {x.stride()}, w {tuple(w.shape)} {w.dtype}")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_skinny_bf16: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    partial, counters, error, stream = _gemm_scratch(x.device, M, N, K)
    pf = None if prefetch is None else _facts(prefetch)
    _check_product("gemm_skinny_bf16", _fn("ts_gemm_skinny_bf16")(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), out.stride(0),
        1 if out.dtype == torch.float32 else 0, partial, counters, error,
        None if pf is None else pf.ptr, 0 if pf is None else min(pf.nbytes, GEMM_PREFETCH_BYTES),
        stream), x, w, out)


_SIGNATURES["ts_gemm_skinny_fused"] = [
    _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_int,
    _c_int, _c_void_p, _c_int, _c_float, _c_float, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p,
]
GEMM_FUSED_MAX_ROWS = 32
GEMM_EPILOGUE_PLAIN, GEMM_EPILOGUE_SWIGLU, GEMM_EPILOGUE_RESIDUAL_NORM = 0, 1, 2


def gemm_skinny_fused(
    x: torch.Tensor,
    w: torch.Tensor,
    *,
    out: Optional[torch.Tensor] = None,
    mode: int = GEMM_EPILOGUE_PLAIN,
    scale_ssq: Optional[torch.Tensor] = None,
    scale_width: int = 1,
    scale_eps: float = 0.0,
    hidden: Optional[torch.Tensor] = None,
    norm_weight: Optional[torch.Tensor] = None,
    xprime: Optional[torch.Tensor] = None,
    ssq_out: Optional[torch.Tensor] = None,
    prefetch: Optional[torch.Tensor] = None,
) -> None:
    """x[M,K] @ w[N,K]^T on the tcgen05 tensor cores (M <= 32) with the work of the neighbouring
    small kernels done where each tile is finished.

    scale_ssq [tiles, M] float32: x lacks its norm's 1/rms (x = source * norm weight); the sums
    of squares of the source rows per 128 columns, as a GEMM in mode 2 leaves them; every row m of
    the product is multiplied by rsqrt(sum_m / scale_width + scale_eps).
    mode GEMM_EPILOGUE_PLAIN: out[M,N] bf16 or float32.
    mode GEMM_EPILOGUE_SWIGLU: the rows of w come in blocks of 128, 64 gate rows and then the 64 up
      rows of the same outputs; out[M,N/2] bf16 = silu(gate) * up.
    mode GEMM_EPILOGUE_RESIDUAL_NORM: hidden[M,N] float32 += product; xprime[M,N] bf16 = hidden *
      norm_weight; ssq_out[ceil(N/128), M] float32 = sums of squares of the new hidden rows.
    """
    if not gemm_skinny_supported(x, w) or x.shape[0] > GEMM_FUSED_MAX_ROWS:
        raise KernelError(
            f"gemm_skinny_fused: needs bfloat16, at most {GEMM_FUSED_MAX_ROWS} rows, K a multiple of 8 and 16-byte "
            f"aligned rows; got x {tuple(x.shape)} {x.dtype} strides {x.stride()}, w {tuple(w.shape)} {w.dtype}")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_skinny_fused: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    ldo, out_f32 = 0, 0
    if mode in (GEMM_EPILOGUE_PLAIN, GEMM_EPILOGUE_SWIGLU):
        cols = N if mode == GEMM_EPILOGUE_PLAIN else N // 2
        if out is None or not out.is_cuda or tuple(out.shape) != (M, cols) or out.stride(1) != 1:
            raise KernelError(f"gemm_skinny_fused: out must be [{M},{cols}]")
        if out.dtype not in ((torch.bfloat16, torch.float32) if mode == GEMM_EPILOGUE_PLAIN else (torch.bfloat16,)):
            raise KernelError(f"gemm_skinny_fused: out dtype {out.dtype} not taken in mode {mode}")
        if mode == GEMM_EPILOGUE_SWIGLU and N % 128:
            raise KernelError("gemm_skinny_fused: the gate/up blocks need N to be a multiple of 128")
        ldo, out_f32 = out.stride(0), 1 if out.dtype == torch.float32 else 0
    elif mode == GEMM_EPILOGUE_RESIDUAL_NORM:
        tiles = -(-N // 128)
        ok = (
            hidden is not None and hidden.dtype == torch.float32 and tuple(hidden.shape) == (M, N) and hidden.is_contiguous()
            and xprime is not None and xprime.dtype == torch.bfloat16 and tuple(xprime.shape) == (M, N) and xprime.is_contiguous()
            and norm_weight is not None and norm_weight.dtype == torch.float32 and norm_weight.numel() == N and norm_weight.is_contiguous()
            and ssq_out is not None and ssq_out.dtype == torch.float32 and ssq_out.numel() >= tiles * M and ssq_out.is_contiguous()
        )
        if not ok:
            raise KernelError("gemm_skinny_fused: mode 2 needs hidden f32 [M,N], xprime bf16 [M,N], norm_weight f32 [N], ssq_out f32 [tiles,M]")
    else:
        raise KernelError(f"gemm_skinny_fused: no mode {mode}")
    scale_tiles = 0
    if scale_ssq is not None:
        if scale_ssq.dtype != torch.float32 or not scale_ssq.is_contiguous() or scale_ssq.dim() != 2 or scale_ssq.shape[1] != M:
            raise KernelError("gemm_skinny_fused: scale_ssq must be float32 [tiles, M]")
        scale_tiles = scale_ssq.shape[0]
    partial, counters, error, stream = _gemm_scratch(x.device, M, N, K)
    pf = None if prefetch is None else _facts(prefetch)
    _check_product("gemm_skinny_fused", _fn("ts_gemm_skinny_fused")(
        x.data_ptr(), w.data_ptr(), _ptr(out), M, N, K, x.stride(0), w.stride(0), ldo, out_f32,
        int(mode), _ptr(scale_ssq), scale_tiles, float(scale_width), float(scale_eps),
        _ptr(hidden), N, _ptr(norm_weight), _ptr(xprime), _ptr(ssq_out),
        partial, counters, error,
        None if pf is None else pf.ptr, 0 if pf is None else min(pf.nbytes, GEMM_PREFETCH_BYTES),
        stream), x, w, out, scale_ssq, hidden, norm_weight, xprime, ssq_out)


_SIGNATURES["ts_gemm_skinny_qk_rope"] = [
    _c_void_p, _c_void_p, _c_int, _c_int, _c_ll, _c_ll, _c_int, _c_int,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
    _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p,
    _c_void_p, _c_int, _c_float, _c_float,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p,
]
GEMM_QK_ROPE_HEAD_DIM = 128

_SIGNATURES["ts_rope_cos_sin"] = [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p]


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """[num_tokens, len(inv_freq), 2] float32: (cos, sin) of positions[t] * inv_freq[j], the float32
    product and functions that the rotating kernels use themselves.  A step computes it once for
    all layers that rotate with the same frequencies."""
    _cuda_contig("positions", positions, torch.int32)
    _cuda_contig("inv_freq", inv_freq, torch.float32)
    if positions.numel() < num_tokens:
        raise KernelError("rope_cos_sin: positions are shorter than the tokens")
    half = inv_freq.numel()
    out = torch.empty((num_tokens, half, 2), device=positions.device, dtype=torch.float32)
    _check("rope_cos_sin", _fn("ts_rope_cos_sin")(positions.data_ptr(), inv_freq.data_ptr(), num_tokens, half, out.data_ptr(), _stream()))
    return out


def gemm_qk_rope_store(
    x: torch.Tensor,
    w: torch.Tensor,
    q_out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    positions: torch.Tensor,
    q_norm_weight: Optional[torch.Tensor],
    k_norm_weight: Optional[torch.Tensor],
    eps: float,
    inv_freq: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    *,
    scale_ssq: Optional[torch.Tensor] = None,
    scale_width: int = 1,
    scale_eps: float = 0.0,
    prefetch: Optional[torch.Tensor] = None,
    cos_sin: Optional[torch.Tensor] = None,
) -> None:
    """The q/k/v projection (w [(nq + 2 nkv) * 128, K], heads of 128) with qk_norm_rope_store's work
    done in the product's epilogue: per-head RMS norm of q and k, rotate-half rotation over the
    whole head (inv_freq [64]) or none, q to q_out [M, nq * 128], k and v to their cache slots.
    At most 32 rows.  scale_ssq as in gemm_skinny_fused.  cos_sin: rope_cos_sin(positions, inv_freq,
    M) if the caller has it (the epilogue then reads the angles' cosines and sines instead of
    computing them)."""
    nq, nkv, d = num_heads, num_kv_heads, GEMM_QK_ROPE_HEAD_DIM
    if not gemm_skinny_supported(x, w) or x.shape[0] > GEMM_FUSED_MAX_ROWS:
        raise KernelError(f"gemm_qk_rope_store: needs bfloat16, at most {GEMM_FUSED_MAX_ROWS} rows and 16-byte aligned rows")
    M, K = x.shape
    if tuple(w.shape) != ((nq + 2 * nkv) * d, K):
        raise KernelError(f"gemm_qk_rope_store: w must be [{(nq + 2 * nkv) * d},{K}], got {tuple(w.shape)}")
    _cuda_contig("q_out", q_out, torch.bfloat16)
    _cuda_contig("k_cache", k_cache, torch.bfloat16)
    _cuda_contig("v_cache", v_cache, torch.bfloat16)
    _cuda_contig("slot_mapping", slot_mapping, torch.int32)
    _cuda_contig("positions", positions, torch.int32)
    if q_out.numel() != M * nq * d or tuple(k_cache.shape[-2:]) != (nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError("gemm_qk_rope_store: q_out must hold [M, nq*128], the caches [.., nkv, 128]")
    if slot_mapping.numel() < M or positions.numel() < M:
        raise KernelError("gemm_qk_rope_store: slot_mapping/positions are shorter than the rows")
    for name, t, n in (("q_norm_weight", q_norm_weight, d), ("k_norm_weight", k_norm_weight, d), ("inv_freq", inv_freq, d // 2)):
        if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or t.numel() != n):
            raise KernelError(f"gemm_qk_rope_store: {name} must be {n} float32 on the device")
    scale_tiles = 0
    if scale_ssq is not None:
        if scale_ssq.dtype != torch.float32 or not scale_ssq.is_contiguous() or scale_ssq.dim() != 2 or scale_ssq.shape[1] != M:
            raise KernelError("gemm_qk_rope_store: scale_ssq must be float32 [tiles, M]")
        scale_tiles = scale_ssq.shape[0]
    if cos_sin is not None and (inv_freq is None or cos_sin.dtype != torch.float32 or not cos_sin.is_cuda or not cos_sin.is_contiguous()
                                or cos_sin.numel() < M * d):
        raise KernelError(f"gemm_qk_rope_store: cos_sin must be float32 [M, {d // 2}, 2] on the device, beside inv_freq")
    partial, counters, error, stream = _gemm_scratch(x.device, M, w.shape[0], K)
    pf = None if prefetch is None else _facts(prefetch)
    _check_product("gemm_qk_rope_store", _fn("ts_gemm_skinny_qk_rope")(
        x.data_ptr(), w.data_ptr(), M, K, x.stride(0), w.stride(0), nq, nkv,
        q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(), positions.data_ptr(),
        _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps), _ptr(inv_freq), _ptr(cos_sin),
        _ptr(scale_ssq), scale_tiles, float(scale_width), float(scale_eps),
        partial, counters, error,
        None if pf is None else pf.ptr, 0 if pf is None else min(pf.nbytes, GEMM_PREFETCH_BYTES),
        stream), x, w, q_out, k_cache, v_cache, slot_mapping, positions, q_norm_weight, k_norm_weight, inv_freq, cos_sin, scale_ssq)


_SIGNATURES["ts_wait_gives_up_probe"] = [_c_void_p, _c_int, _c_void_p]


def wait_gives_up_probe(device: torch.device, limit: int = 4096) -> None:
    """Launches a kernel whose only bounded wait runs out (an mbarrier nothing feeds, `limit`
    tries) and which then raises the current stream's error word exactly as the tcgen05 kernels
    do: the way to see the error path work without a fault.  check_device_errors() raises after
    the next synchronisation."""
    flush_gemm_chain()
    _, error = _gemm_workspace(device)
    _check("wait_gives_up_probe", _fn("ts_wait_gives_up_probe")(error.data_ptr(), int(limit), _stream()))


def library_mm(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None, float32_out: bool = False) -> torch.Tensor:
    """x [T, in] @ weight[out, in]^T by the library GEMM (cuBLAS through torch.mm), for steps of more
    rows than the engine's own weight-streaming kernel takes; a float32 result keeps the sums
    unrounded (the logits)."""
    flush_gemm_chain()  # the library reads x by itself
    if float32_out:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    return torch.mm(x, weight.t(), out=out)


# Timers per kernel class, for eager steps (a replayed graph has no calls to time): switched on,
# every launching function of this module is wrapped so that a pair of CUDA events brackets what it
# launches; switched off, the functions are the plain ones again and nothing is paid.
_TIMED = ("embed_gather", "feed_tokens", "add_rmsnorm", "residual_add", "swiglu", "qk_norm_rope_store", "attention_paged_simple",
          "sample", "sgemm_nt", "attention_paged_mma", "attention_decode_flat", "attention_prefill_tcgen05", "gemm_skinny_bf16",
          "gemm_skinny_fused", "rope_cos_sin", "gemm_qk_rope_store", "library_mm")
_plain_functions: dict[str, object] = {}
_kernel_events: list[tuple[str, "torch.cuda.Event", "torch.cuda.Event"]] = []


def time_kernels(on: bool) -> None:
    """Switches the per-class timers on or off (see kernel_times)."""
    import functools

    g = globals()
    if on and not _plain_functions:
        for name in _TIMED:
            plain = g[name]

            def timed(*args, _plain=plain, _name=name, **kwargs):
                if torch.cuda.is_current_stream_capturing():
                    return _plain(*args, **kwargs)
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                result = _plain(*args, **kwargs)
                stop.record()
                _kernel_events.append((_name, start, stop))
                return result

            _plain_functions[name] = plain
            g[name] = functools.wraps(plain)(timed)
    elif not on and _plain_functions:
        for name, plain in _plain_functions.items():
            g[name] = plain
        _plain_functions.clear()


def kernel_times() -> dict[str, dict]:
    """{function: {"calls": n, "ms": device time between the events around its launches}} since the
    last call, after waiting for the device.  Classes: the function names of this module
    (`gemm_skinny_fused` includes the norms and activations folded into it; `library_mm` is cuBLAS)."""
    torch.cuda.synchronize()
    out: dict[str, dict] = {}
    for name, start, stop in _kernel_events:
        row = out.setdefault(name, {"calls": 0, "ms": 0.0})
        row["calls"] += 1
        row["ms"] += start.elapsed_time(stop)
    _kernel_events.clear()
    for row in out.values():
        row["ms"] = round(row["ms"], 3)
    return out


def check_device_errors() -> None:
    """Raises if a kernel reported that one of its bounded waits gave up.  Cheap: reads
    pinned host words; call it wherever the host has just synchronised anyway."""
    if _attention_error is not None and _word_is_set(_attention_error):
        raise KernelError("decode attention: a wait on an mbarrier gave up (the kernel returned early)")
    for (dev, _), (_, error) in _gemm_workspaces.items():
        if _word_is_set(error):
            raise KernelError(f"a tcgen05 kernel on cuda:{dev} (skinny GEMM or prompt attention): a wait on an mbarrier gave up (the kernel returned early)")

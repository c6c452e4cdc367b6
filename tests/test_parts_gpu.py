"""Each part alone against the plain functions, and the generality of the layer machinery:
a toy mixer with state of its own, a layer that runs twice, a layer that reads another's cache.
The toy parts are defined here; no file of the framework changes for them."""

from dataclasses import asdict, dataclass

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.replay_helpers import replay_in_process, trace_decode_tail, trace_mixed, trace_portions, trace_whole

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def ctx(dtype):
    from tokensprint_b200.parts.base import BuildContext

    return BuildContext(device=torch.device(DEV), dtype=dtype)


def one_sequence_step(T, page, dtype, start=0):
    """A StepContext for one sequence of T tokens at positions start..start+T-1, pages 3, 1, 4, ... ."""
    from tokensprint_b200.parts.base import GroupTables, StepContext

    n_pages = -(-(start + T) // page)
    table = [(7 * i + 3) % (n_pages + 5) for i in range(n_pages)]
    assert len(set(table)) == n_pages
    slots = [table[p // page] * page + p % page for p in range(start, start + T)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    step = StepContext(
        num_tokens=T, num_seqs=1, token_ids=i32([0] * T), positions=i32(list(range(start, start + T))),
        seq_index=i32([0] * T), cu_seqlens_q=i32([0, T]), context_lens=i32([start + T]), state_slots=i32([0]),
        groups=[GroupTables(block_table=i32([table]), slot_mapping=i32(slots))], page_size=page,
        max_seqlen_q=T, max_context_len=start + T, host_seq_starts=[start], host_seq_lens=[T], host_state_slots=[0])
    return step, n_pages + 5


TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from tokensprint_b200.parts.base import PartSpec, build_part

    H, T, eps = 200, 6, 1e-4
    norm = build_part("norm", PartSpec("rmsnorm", {"dim": H, "eps": eps, "weight": "w"}), ctx(dtype))
    assert [(s.name, s.shape, s.role) for s in norm.tensor_specs()] == [("w", (H,), "vector")]
    w = 1 + 0.1 * torch.randn(H, device=DEV)
    norm.load({"w": w})
    hidden = torch.randn(T, H, device=DEV)
    delta = torch.randn(T, H, device=DEV).to(dtype)
    want_h = hidden.double() + delta.double()
    out = torch.empty(T, H, device=DEV, dtype=dtype)
    norm.forward(hidden, delta, out)
    assert rel_err(hidden, want_h) < 1e-6
    assert rel_err(out, plain.rms_norm(want_h.cpu(), w.double().cpu(), eps)) < TOL[dtype]


def test_position_part_owns_the_reference_frequencies():
    from tokensprint_b200.parts.base import PartSpec, build_part

    rope = build_part("position_encoding", PartSpec("rotary", {"dim": 48, "theta": 5e4}), ctx(torch.float32))
    assert torch.equal(rope.rotary_inv_freq().cpu(), plain.rope_inverse_frequencies(48, 5e4))
    with pytest.raises(ValueError):
        build_part("position_encoding", PartSpec("rotary", {"dim": 7, "theta": 1e4}), ctx(torch.float32))


def test_position_part_makes_a_step_s_cosines_and_sines_once():
    """The table that the fused q/k/v product reads: the reference's angles (float32 position times
    float32 inverse frequency), made by the first layer that asks in a step, found again by a part
    with the same width and base, not by one with another base, and not kept for the next run."""
    from tokensprint_b200.parts.base import PartSpec, build_part

    step, _ = one_sequence_step(11, 8, torch.float32, start=1000)
    a = build_part("position_encoding", PartSpec("rotary", {"dim": 128, "theta": 1e6}), ctx(torch.bfloat16))
    b = build_part("position_encoding", PartSpec("rotary", {"dim": 128, "theta": 1e6}), ctx(torch.bfloat16))
    c = build_part("position_encoding", PartSpec("rotary", {"dim": 128, "theta": 1e4}), ctx(torch.bfloat16))
    table = a.rotary_cos_sin(step)
    angles = plain.rope_angles(list(range(1000, 1011)), 128, 1e6)  # [T, 64] float32
    assert table.shape == (11, 64, 2) and table.dtype == torch.float32
    assert float((table[..., 0].cpu().double() - torch.cos(angles.double())).abs().max()) < 1e-6
    assert float((table[..., 1].cpu().double() - torch.sin(angles.double())).abs().max()) < 1e-6
    assert b.rotary_cos_sin(step) is table
    assert c.rotary_cos_sin(step) is not table
    step.shared.clear()  # what a model does before it runs its blocks again
    again = a.rotary_cos_sin(step)
    assert again is not table and torch.equal(again, table)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from tokensprint_b200.parts.base import PartSpec, build_part

    H, I, T = 72, 104, 9
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I, "gate": "g", "up": "u", "down": "d"}), ctx(dtype))
    assert {s.name: s.shape for s in ffn.tensor_specs()} == {"g": (I, H), "u": (I, H), "d": (H, I)}
    w = {"g": torch.randn(I, H) * 0.2, "u": torch.randn(I, H) * 0.2, "d": torch.randn(H, I) * 0.2}
    ffn.load({k: v.to(DEV, dtype) for k, v in w.items()})
    x = torch.randn(T, H)
    got = ffn.forward(x.to(DEV, dtype), None)
    wd = {f"p.{k}_proj.weight": v.to(dtype).double() for k, v in (("gate", w["g"]), ("up", w["u"]), ("down", w["d"]))}
    want = plain.swiglu_ffn(x.to(dtype).double(), wd, "p.")
    assert rel_err(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 10])
def test_attention_part_and_block(dtype, window):
    """The attention mixer alone (prefill of a portion that starts mid-sequence is covered by the
    replay tests; here one whole sequence), then a whole pre-norm block around it."""
    from tokensprint_b200.parts.base import LayerCache, PartSpec, build_part

    H, nq, nkv, d, I, T, page, eps, theta = 80, 6, 2, 32, 96, 37, 8, 1e-5, 1e4
    names = {k: f"a.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
    mixer_spec = PartSpec("attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "qk_norm": True,
                                        "qk_norm_eps": eps, "window": window, "position": PartSpec("rotary", {"dim": d, "theta": theta}), **names})
    g = torch.Generator().manual_seed(3)
    w = {"a.q": torch.randn(nq * d, H, generator=g) * 0.2, "a.k": torch.randn(nkv * d, H, generator=g) * 0.2,
         "a.v": torch.randn(nkv * d, H, generator=g) * 0.2, "a.o": torch.randn(H, nq * d, generator=g) * 0.2,
         "a.q_norm": 1 + 0.1 * torch.randn(d, generator=g), "a.k_norm": 1 + 0.1 * torch.randn(d, generator=g),
         "f.g": torch.randn(I, H, generator=g) * 0.2, "f.u": torch.randn(I, H, generator=g) * 0.2, "f.d": torch.randn(H, I, generator=g) * 0.2,
         "n1": 1 + 0.1 * torch.randn(H, generator=g), "n2": 1 + 0.1 * torch.randn(H, generator=g)}
    dev_w = {k: (v.to(DEV) if v.dim() == 1 else v.to(DEV, dtype)) for k, v in w.items()}
    pw = {}
    for k, v in w.items():
        v = v.double() if v.dim() == 1 else v.to(dtype).double()
        pw[{"a.q": "p.self_attn.q_proj.weight", "a.k": "p.self_attn.k_proj.weight", "a.v": "p.self_attn.v_proj.weight",
            "a.o": "p.self_attn.o_proj.weight", "a.q_norm": "p.self_attn.q_norm.weight", "a.k_norm": "p.self_attn.k_norm.weight",
            "f.g": "p.mlp.gate_proj.weight", "f.u": "p.mlp.up_proj.weight", "f.d": "p.mlp.down_proj.weight",
            "n1": "p.input_layernorm.weight", "n2": "p.post_attention_layernorm.weight"}[k]] = v

    step, n_pages = one_sequence_step(T, page, dtype)
    cache = LayerCache(group=0, k_pages=torch.zeros(n_pages, page, nkv, d, device=DEV, dtype=dtype),
                       v_pages=torch.zeros(n_pages, page, nkv, d, device=DEV, dtype=dtype))
    mixer = build_part("mixer", mixer_spec, ctx(dtype))
    need = mixer.cache_need()
    assert (need.kind, need.window, need.kv_heads, need.head_dim) == ("window" if window else "full", window, nkv, d)
    mixer.load(dev_w)
    x = torch.randn(T, H, generator=g)
    got = mixer.forward(x.to(DEV, dtype), step, cache)
    want = plain.attention_layer(x.to(dtype).double(), pw, "p.self_attn.", list(range(T)), num_heads=nq, num_kv_heads=nkv,
                                 head_dim=d, rope_theta=theta, eps=eps, window=window or None)
    assert rel_err(got, want) < TOL[dtype]

    block = build_part("block", PartSpec("pre_norm", {
        "mixer": mixer_spec,
        "feed_forward": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I, "gate": "f.g", "up": "f.u", "down": "f.d"}),
        "mixer_norm": PartSpec("rmsnorm", {"dim": H, "eps": eps, "weight": "n1"}),
        "ffn_norm": PartSpec("rmsnorm", {"dim": H, "eps": eps, "weight": "n2"})}), ctx(dtype))
    block.load(dev_w)
    hidden = torch.randn(T, H, generator=g).to(DEV)
    h0 = hidden.double().cpu()
    pending = block.forward(hidden, None, step, cache)
    cfg = {"rms_norm_eps": eps, "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "rope_theta": theta}
    pw2 = {"model.layers.0." + k[2:]: v for k, v in pw.items()}
    want_h = plain.block(h0, pw2, 0, list(range(T)), cfg, window or None)
    assert rel_err(hidden.double().cpu() + pending.double().cpu(), want_h) < TOL[dtype]


# ---------------------------------------------------------------------------
# a toy architecture defined here: attention layers beside a mixer with per-request state


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = 48
    num_hidden_layers: int = 3
    intermediate_size: int = 64
    rms_norm_eps: float = 1e-5
    architectures: tuple = ("ToyStateForCausalLM",)

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        return d

    def save(self, folder):
        import json
        from pathlib import Path

        Path(folder).mkdir(parents=True, exist_ok=True)
        (Path(folder) / "config.json").write_text(json.dumps(self.to_dict()))


def _register_toy():
    from tokensprint_b200.config.registry import register_architecture
    from tokensprint_b200.models.spec import ModelSpec
    from tokensprint_b200.parts.base import CacheNeed, Mixer, PartSpec, TensorSpec, register_part

    @register_part("mixer", "toy_running_mean", replace=True)
    class RunningMeanMixer(Mixer):
        """y_t = W * mean(x_0 .. x_t).  Its cache is no page at all but one slot per request:
        the running sum of the inputs and their count (width + 1 floats)."""

        def __init__(self, bctx, *, hidden_size, weight):
            self.H, self.weight_name, self.dtype = hidden_size, weight, bctx.dtype
            self.weight = None

        def cache_need(self):
            return CacheNeed(kind="none", state_shape=(self.H + 1,), state_dtype=torch.float32)

        def tensor_specs(self):
            return [TensorSpec(self.weight_name, (self.H, self.H))]

        def load(self, tensors):
            self.weight = tensors[self.weight_name]

        def forward(self, x, step, cache):
            out = torch.empty_like(x)
            t0 = 0
            for n, slot in zip(step.host_seq_lens, step.host_state_slots):
                state = cache.state[slot]
                sums = state[: self.H] + torch.cumsum(x[t0 : t0 + n].float(), dim=0)
                counts = state[self.H] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[t0 : t0 + n] = ((sums / counts[:, None]).to(x.dtype) @ self.weight.t())
                state[: self.H] = sums[-1]
                state[self.H] = counts[-1]
                t0 += n
            return out

    @register_architecture("ToyStateForCausalLM", config_from_dict=lambda d: ToyConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items()}))
    def build_toy(cfg: ToyConfig):
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"toy.{i}."
            if i % 2 == 0:
                mixer = PartSpec("toy_running_mean", {"hidden_size": cfg.hidden_size, "weight": p + "mix.weight"})
            else:
                mixer = PartSpec("attention", {"hidden_size": cfg.hidden_size, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                                               "position": PartSpec("rotary", {"dim": 16, "theta": 1e4}),
                                               "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"})
            norm = {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps}
            layers.append(PartSpec("pre_norm", {
                "mixer": mixer,
                "feed_forward": PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                                                    "gate": p + "gate", "up": p + "up", "down": p + "down"}),
                "mixer_norm": PartSpec("rmsnorm", {**norm, "weight": p + "n1"}),
                "ffn_norm": PartSpec("rmsnorm", {**norm, "weight": p + "n2"})}))
        return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, embedding="toy.embed", layers=layers,
                         final_norm=PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps, "weight": "toy.norm"}),
                         lm_head="toy.head", max_positions=512)


def _plain_toy(weights, cfg: ToyConfig, ids):
    w = {k: v.double() for k, v in weights.items()}
    T = len(ids)
    h = plain.embedding(w["toy.embed"], ids)
    for i in range(cfg.num_hidden_layers):
        p = f"toy.{i}."
        x = plain.rms_norm(h, w[p + "n1"], cfg.rms_norm_eps)
        if i % 2 == 0:
            mean = torch.cumsum(x, dim=0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
            a = mean @ w[p + "mix.weight"].T
        else:
            q = (x @ w[p + "q"].T).view(T, 3, 16)
            k = (x @ w[p + "k"].T).view(T, 1, 16)
            v = (x @ w[p + "v"].T).view(T, 1, 16)
            ang = plain.rope_angles(range(T), 16, 1e4)
            o = plain.causal_attention(plain.apply_rope(q, ang), plain.apply_rope(k, ang), v, scale=16**-0.5)
            a = o.reshape(T, 48) @ w[p + "o"].T
        h = h + a
        x = plain.rms_norm(h, w[p + "n2"], cfg.rms_norm_eps)
        g, u = x @ w[p + "gate"].T, x @ w[p + "up"].T
        h = h + (g * torch.sigmoid(g) * u) @ w[p + "down"].T
    return plain.rms_norm(h, w["toy.norm"], cfg.rms_norm_eps) @ w["toy.head"].T


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from tokensprint_b200.config.registry import unregister_architecture
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.parts.base import unregister_part
    from tokensprint_b200.weights.loader import write_random_model
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    _register_toy()
    try:
        cfg = ToyConfig()
        folder = write_random_model(tmp_path / "toy", cfg, seed=4, dtype="float32", std=0.15)
        files = SafetensorsFolder(folder)
        weights = {n: files.tensor(n).clone() for n in files.keys()}
        assert "toy.0.mix.weight" in weights and "toy.1.q" in weights
        g = torch.Generator().manual_seed(8)
        requests = {f"r{i}": torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((3, 20, 41, 64))}
        want = {rid: _plain_toy(weights, cfg, ids) for rid, ids in requests.items()}
        many = dict(requests)
        many.update({k + "x": v for k, v in requests.items()})
        for steps, reqs in ((trace_whole(requests), requests), (trace_decode_tail(requests, 16), requests),
                            (trace_portions(requests), requests), (trace_mixed(many, 256, seed=3), many)):
            replayer = TraceReplayer.from_folder(folder, "float32", 256)
            runner = replayer.runner
            assert [g.kind for g in runner.groups] == ["full"]  # one page group; the toy mixer has none
            assert runner.cache_tensors.state[0] is not None and runner.cache_tensors.k[0] is None
            assert not runner.use_graphs
            got = replay_in_process(replayer, steps)
            for (rid, pos), row in got.items():
                ref = want[rid.rstrip("x")][pos].numpy()
                assert abs(row - ref).max() < 1e-4 * abs(want[rid.rstrip("x")]).max(), f"{rid} position {pos}"
            assert len(got) == sum(len(v) for v in reqs.values())
    finally:
        unregister_architecture("ToyStateForCausalLM")
        unregister_part("mixer", "toy_running_mean")


def test_run_order_is_data_a_layer_twice_and_a_shared_cache(tmp_path):
    """Run order: layer 0, layer 1, layer 0 again (own cache), layer 2 reading layer 1's cache."""
    from tests.tiny_configs import TINY_B, tiny_weights, write_model_folder
    from tokensprint_b200.models.qwen3 import Qwen3Config
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.engine.runner import ModelRunner
    from tokensprint_b200.models.model import Model
    from tokensprint_b200.models.qwen3 import build_qwen3_spec
    from tokensprint_b200.models.spec import RunSpec
    from tokensprint_b200.weights.loader import FolderSource

    cfg = TINY_B
    weights = tiny_weights(cfg, 21, std=0.05, sharp=2.0)
    folder = write_model_folder(tmp_path / "m", cfg, weights)
    spec = build_qwen3_spec(Qwen3Config.from_dict(cfg))
    spec.run_order = [RunSpec(0), RunSpec(1, cache=7), RunSpec(0), RunSpec(2, cache=7, writes_cache=False)]
    model = Model(spec, DEV, torch.float32)
    assert len(model.cache_plan) == 3 and model.run_cache == [0, 1, 2, 1]
    model.load(FolderSource(folder))
    runner = ModelRunner(model, page_size=16, num_pages=32, num_slots=4)

    # plain: the same order; the last run attends with its own queries over layer 1's keys and values
    w = {k: v.double() for k, v in weights.items()}
    ids = torch.randint(0, cfg["vocab_size"], (45,), generator=torch.Generator().manual_seed(2)).tolist()
    T, pos = len(ids), list(range(len(ids)))
    nq, nkv, d, eps, theta = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"], cfg["rope_theta"]
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    h = plain.block(h, w, 0, pos, cfg, None)
    x1 = plain.rms_norm(h, w["model.layers.1.input_layernorm.weight"], eps)
    ang = plain.rope_angles(pos, d, theta)
    k1 = plain.apply_rope(plain.rms_norm((x1 @ w["model.layers.1.self_attn.k_proj.weight"].T).view(T, nkv, d), w["model.layers.1.self_attn.k_norm.weight"], eps), ang)
    v1 = (x1 @ w["model.layers.1.self_attn.v_proj.weight"].T).view(T, nkv, d)
    h = plain.block(h, w, 1, pos, cfg, None)
    h = plain.block(h, w, 0, pos, cfg, None)
    p = "model.layers.2."
    x2 = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps)
    q2 = plain.apply_rope(plain.rms_norm((x2 @ w[p + "self_attn.q_proj.weight"].T).view(T, nq, d), w[p + "self_attn.q_norm.weight"], eps), ang)
    a = plain.causal_attention(q2, k1, v1, scale=d**-0.5).reshape(T, nq * d) @ w[p + "self_attn.o_proj.weight"].T
    h = h + a
    h = h + plain.swiglu_ffn(plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    want = plain.rms_norm(h, w["model.norm.weight"], eps) @ w["lm_head.weight"].T

    for steps in (trace_whole({"a": ids}), trace_portions({"a": ids}), trace_decode_tail({"a": ids}, 20)):
        got = replay_in_process(TraceReplayer(runner), steps)
        for (rid, position), row in got.items():
            assert abs(row - want[position].numpy()).max() < 1e-4 * float(want.abs().max()), f"position {position}"
    assert runner.cache_manager.pages_in_use() == 0


# ---------------------------------------------------------------------------
# two more toy parts defined here: a feed-forward with routing and a position encoding with a
# table of its own (never a model of anyone's: they only show that the interfaces suffice)


@dataclass(frozen=True)
class ToyRoutedConfig:
    vocab_size: int = 61
    hidden_size: int = 40
    num_hidden_layers: int = 2
    num_experts: int = 3
    expert_size: int = 24
    max_positions: int = 96
    rms_norm_eps: float = 1e-6
    architectures: tuple = ("ToyRoutedForCausalLM",)

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        return d

    def save(self, folder):
        import json
        from pathlib import Path

        Path(folder).mkdir(parents=True, exist_ok=True)
        (Path(folder) / "config.json").write_text(json.dumps(self.to_dict()))


def _register_routed_toy():
    from tokensprint_b200.config.registry import register_architecture
    from tokensprint_b200.models.spec import ModelSpec
    from tokensprint_b200.parts.base import FeedForward, PartSpec, PositionEncoding, TensorSpec, register_part

    @register_part("feed_forward", "toy_top1_experts", replace=True)
    class Top1Experts(FeedForward):
        """Each token goes to the expert its router row scores highest, y = p_e * W2_e relu(W1_e x),
        p the softmax of the router scores (float32).  The tokens of an expert are gathered on the
        host's say-so, so a step of it is not a fixed sequence of kernels: graph_safe stays False."""

        def __init__(self, bctx, *, hidden_size, expert_size, num_experts, prefix):
            self.H, self.I, self.E, self.prefix = hidden_size, expert_size, num_experts, prefix

        def tensor_specs(self):
            specs = [TensorSpec(self.prefix + "router", (self.E, self.H), "vector")]  # routing in float32
            for e in range(self.E):
                specs += [TensorSpec(f"{self.prefix}{e}.w1", (self.I, self.H)), TensorSpec(f"{self.prefix}{e}.w2", (self.H, self.I))]
            return specs

        def load(self, tensors):
            self.router = tensors[self.prefix + "router"]
            self.w1 = [tensors[f"{self.prefix}{e}.w1"] for e in range(self.E)]
            self.w2 = [tensors[f"{self.prefix}{e}.w2"] for e in range(self.E)]

        def forward(self, x, step):
            probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
            top_p, top_e = probs.max(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.E):
                rows = (top_e == e).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(x[rows] @ self.w1[e].t()) @ self.w2[e].t()
                    out[rows] = (y.float() * top_p[rows, None]).to(x.dtype)
            return out

    @register_part("position_encoding", "toy_learned_offsets", replace=True)
    class LearnedOffsets(PositionEncoding):
        """q and k get a learned row of a table added, by position: an encoding the fused kernel
        does not know, so the attention mixer norms, calls `apply`, then stores."""

        graph_safe = True  # one gather and two adds on device values

        def __init__(self, bctx, *, dim, max_positions, table):
            self.dim, self.max_positions, self.table_name = dim, max_positions, table

        def tensor_specs(self):
            return [TensorSpec(self.table_name, (self.max_positions, self.dim))]

        def load(self, tensors):
            self.table = tensors[self.table_name]

        def apply(self, q, k, step):
            rows = self.table[step.positions.long()]
            q += rows[:, None, :]
            k += rows[:, None, :]

    @register_architecture("ToyRoutedForCausalLM", config_from_dict=lambda d: ToyRoutedConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items()}))
    def build(cfg: ToyRoutedConfig):
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"m.{i}."
            mixer = PartSpec("attention", {"hidden_size": cfg.hidden_size, "num_heads": 4, "num_kv_heads": 2, "head_dim": 8,
                                           "position": PartSpec("toy_learned_offsets", {"dim": 8, "max_positions": cfg.max_positions, "table": p + "pos"}),
                                           "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"})
            norm = {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps}
            layers.append(PartSpec("pre_norm", {
                "mixer": mixer,
                "feed_forward": PartSpec("toy_top1_experts", {"hidden_size": cfg.hidden_size, "expert_size": cfg.expert_size,
                                                              "num_experts": cfg.num_experts, "prefix": p + "experts."}),
                "mixer_norm": PartSpec("rmsnorm", {**norm, "weight": p + "n1"}),
                "ffn_norm": PartSpec("rmsnorm", {**norm, "weight": p + "n2"})}))
        return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, embedding="m.embed", layers=layers,
                         final_norm=PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps, "weight": "m.norm"}),
                         lm_head="m.head", max_positions=cfg.max_positions)


def _plain_routed_toy(weights, cfg: ToyRoutedConfig, ids):
    w = {k: v.double() for k, v in weights.items()}
    T = len(ids)
    h = plain.embedding(w["m.embed"], ids)
    for i in range(cfg.num_hidden_layers):
        p = f"m.{i}."
        x = plain.rms_norm(h, w[p + "n1"], cfg.rms_norm_eps)
        off = w[p + "pos"][:T]
        q = (x @ w[p + "q"].T).view(T, 4, 8) + off[:, None, :]
        k = (x @ w[p + "k"].T).view(T, 2, 8) + off[:, None, :]
        v = (x @ w[p + "v"].T).view(T, 2, 8)
        h = h + plain.causal_attention(q, k, v, scale=8**-0.5).reshape(T, 32) @ w[p + "o"].T
        x = plain.rms_norm(h, w[p + "n2"], cfg.rms_norm_eps)
        probs = torch.softmax(x @ w[p + "experts.router"].T, dim=-1)
        y = torch.zeros_like(x)
        for t in range(T):
            e = int(probs[t].argmax())
            y[t] = probs[t, e] * (torch.relu(x[t] @ w[f"{p}experts.{e}.w1"].T) @ w[f"{p}experts.{e}.w2"].T)
        h = h + y
    return plain.rms_norm(h, w["m.norm"], cfg.rms_norm_eps) @ w["m.head"].T


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding(tmp_path):
    """Registered here, built from config.json and stepped in every way of cutting, without a
    change to the framework's files; the model reports that its decode steps cannot be graphs."""
    from tokensprint_b200.config.registry import unregister_architecture
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.parts.base import unregister_part
    from tokensprint_b200.weights.loader import write_random_model
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    _register_routed_toy()
    try:
        cfg = ToyRoutedConfig()
        folder = write_random_model(tmp_path / "routed", cfg, seed=11, dtype="float32", std=0.2)
        files = SafetensorsFolder(folder)
        weights = {n: files.tensor(n).clone() for n in files.keys()}
        assert "m.0.experts.router" in weights and "m.1.pos" in weights and "m.0.experts.2.w2" in weights
        g = torch.Generator().manual_seed(5)
        requests = {f"r{i}": torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((2, 17, 40, 70))}
        want = {rid: _plain_routed_toy(weights, cfg, ids) for rid, ids in requests.items()}
        # every expert is used by some token, so the routing is exercised
        many = dict(requests)
        many.update({k + "x": v for k, v in requests.items()})
        for steps, reqs in ((trace_whole(requests), requests), (trace_decode_tail(requests, 16), requests),
                            (trace_portions(requests), requests), (trace_mixed(many, 320, seed=6), many)):
            replayer = TraceReplayer.from_folder(folder, "float32", 320)
            assert not replayer.runner.model.graph_safe
            assert replayer.runner.model.blocks[0].mixer.graph_safe  # the attention with the toy encoding alone could be
            got = replay_in_process(replayer, steps)
            for (rid, pos), row in got.items():
                ref = want[rid.rstrip("x")][pos].numpy()
                assert abs(row - ref).max() < 1e-4 * abs(want[rid.rstrip("x")]).max(), f"{rid} position {pos}"
            assert len(got) == sum(len(v) for v in reqs.values())
    finally:
        unregister_architecture("ToyRoutedForCausalLM")
        unregister_part("feed_forward", "toy_top1_experts")
        unregister_part("position_encoding", "toy_learned_offsets")


# ---------------------------------------------------------------------------
# a toy norm and a toy arrangement of a block, again defined here (the two kinds of part that the
# toys above took from the framework)


@dataclass(frozen=True)
class ToyParallelConfig:
    vocab_size: int = 53
    hidden_size: int = 48
    num_hidden_layers: int = 3
    intermediate_size: int = 40
    max_positions: int = 128
    norm_eps: float = 3e-5
    architectures: tuple = ("ToyParallelForCausalLM",)

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        return d

    def save(self, folder):
        import json
        from pathlib import Path

        Path(folder).mkdir(parents=True, exist_ok=True)
        (Path(folder) / "config.json").write_text(json.dumps(self.to_dict()))


def _register_parallel_toy():
    from tokensprint_b200.config.registry import register_architecture
    from tokensprint_b200.models.spec import ModelSpec
    from tokensprint_b200.parts.base import Block, Norm, PartSpec, TensorSpec, build_part, register_part

    @register_part("norm", "toy_centered", replace=True)
    class CenteredNorm(Norm):
        """y = (x - mean x) * rsqrt(var x + eps) * weight + bias: a norm that subtracts the mean and
        has a bias, so nobody can fold it into a product (params() stays None)."""

        graph_safe = True  # a fixed sequence of device operations

        def __init__(self, bctx, *, dim, eps, weight, bias):
            self.dim, self.eps, self.weight_name, self.bias_name = dim, eps, weight, bias

        def tensor_specs(self):
            return [TensorSpec(self.weight_name, (self.dim,), "vector"), TensorSpec(self.bias_name, (self.dim,), "vector")]

        def load(self, tensors):
            self.weight, self.bias = tensors[self.weight_name], tensors[self.bias_name]

        def forward(self, hidden, delta, out, row_index=None):
            if delta is not None:
                hidden += delta.float()
            rows = hidden if row_index is None else hidden[row_index.long()[: out.shape[0]]]
            centred = rows - rows.mean(dim=-1, keepdim=True)
            out.copy_((centred * torch.rsqrt(centred.square().mean(dim=-1, keepdim=True) + self.eps) * self.weight + self.bias).to(out.dtype))

    @register_part("block", "toy_parallel", replace=True)
    class ParallelBlock(Block):
        """h = h + Mixer(N(h)) + FeedForward(N(h)): one norm, both branches read it, their sum is the
        block's pending output."""

        def __init__(self, bctx, *, mixer, feed_forward, norm):
            self.dtype = bctx.dtype
            self.mixer = build_part("mixer", mixer, bctx)
            self.feed_forward = build_part("feed_forward", feed_forward, bctx)
            self.norm = build_part("norm", norm, bctx)
            self._parts = (self.norm, self.mixer, self.feed_forward)
            self.graph_safe = all(p.graph_safe for p in self._parts)

        def tensor_specs(self):
            return [s for p in self._parts for s in p.tensor_specs()]

        def load(self, tensors):
            for p in self._parts:
                p.load(tensors)

        def forward(self, hidden, pending, step, cache):
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            self.norm.forward(hidden, pending, x)
            return self.mixer.forward(x, step, cache) + self.feed_forward.forward(x, step)

        def first_weight(self):
            return self.mixer.first_weight()

    @register_architecture("ToyParallelForCausalLM", config_from_dict=lambda d: ToyParallelConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items()}))
    def build(cfg: ToyParallelConfig):
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"t.{i}."
            mixer = PartSpec("attention", {"hidden_size": cfg.hidden_size, "num_heads": 6, "num_kv_heads": 3, "head_dim": 16,
                                           "position": PartSpec("rotary", {"dim": 16, "theta": 500.0}),
                                           "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"})
            ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                                      "gate": p + "g", "up": p + "u", "down": p + "d"})
            layers.append(PartSpec("toy_parallel", {"mixer": mixer, "feed_forward": ffn,
                                                    "norm": PartSpec("toy_centered", {"dim": cfg.hidden_size, "eps": cfg.norm_eps, "weight": p + "nw", "bias": p + "nb"})}))
        return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, embedding="t.embed", layers=layers,
                         final_norm=PartSpec("toy_centered", {"dim": cfg.hidden_size, "eps": cfg.norm_eps, "weight": "t.nw", "bias": "t.nb"}),
                         lm_head="t.head", max_positions=cfg.max_positions)


def _plain_parallel_toy(weights, cfg: ToyParallelConfig, ids):
    w = {k: v.double() for k, v in weights.items()}
    T = len(ids)

    def centred_norm(x, weight, bias):
        c = x - x.mean(dim=-1, keepdim=True)
        return c * torch.rsqrt(c.square().mean(dim=-1, keepdim=True) + cfg.norm_eps) * weight + bias

    h = plain.embedding(w["t.embed"], ids)
    angles = plain.rope_angles(list(range(T)), 16, 500.0)
    for i in range(cfg.num_hidden_layers):
        p = f"t.{i}."
        x = centred_norm(h, w[p + "nw"], w[p + "nb"])
        q = plain.apply_rope((x @ w[p + "q"].T).view(T, 6, 16), angles)
        k = plain.apply_rope((x @ w[p + "k"].T).view(T, 3, 16), angles)
        v = (x @ w[p + "v"].T).view(T, 3, 16)
        attn = plain.causal_attention(q, k, v, scale=16**-0.5).reshape(T, 96) @ w[p + "o"].T
        gate = x @ w[p + "g"].T
        ffn = (gate * torch.sigmoid(gate) * (x @ w[p + "u"].T)) @ w[p + "d"].T
        h = h + attn + ffn
    return centred_norm(h, w["t.nw"], w["t.nb"]) @ w["t.head"].T


def test_a_toy_norm_and_a_toy_arrangement_of_a_block(tmp_path):
    """A norm with a mean and a bias and a block whose two branches read one norm, registered here,
    around the framework's own attention and SwiGLU parts: built from config.json and stepped in
    every way of cutting, eager and (the parts being fixed sequences of device work) in graphs."""
    from tokensprint_b200.config.registry import unregister_architecture
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.parts.base import unregister_part
    from tokensprint_b200.weights.loader import write_random_model
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    _register_parallel_toy()
    try:
        cfg = ToyParallelConfig()
        folder = write_random_model(tmp_path / "parallel", cfg, seed=23, dtype="float32", std=0.2)
        files = SafetensorsFolder(folder)
        weights = {n: files.tensor(n).clone() for n in files.keys()}
        assert "t.1.nb" in weights and "t.nb" in weights and weights["t.0.nw"].dtype == torch.float32
        g = torch.Generator().manual_seed(9)
        requests = {f"r{i}": torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((3, 19, 45, 66))}
        want = {rid: _plain_parallel_toy(weights, cfg, ids) for rid, ids in requests.items()}
        many = dict(requests)
        many.update({k + "x": v for k, v in requests.items()})
        for steps, reqs, graphs in ((trace_whole(requests), requests, False), (trace_decode_tail(requests, 16), requests, False),
                                    (trace_decode_tail(requests, 16), requests, True), (trace_portions(requests), requests, False),
                                    (trace_mixed(many, 320, seed=4), many, True)):
            replayer = TraceReplayer.from_folder(folder, "float32", 320, graphs=graphs)
            assert replayer.runner.model.graph_safe
            got = replay_in_process(replayer, steps)
            assert not graphs or replayer.runner._graphs
            for (rid, pos), row in got.items():
                ref = want[rid.rstrip("x")][pos].numpy()
                assert abs(row - ref).max() < 1e-4 * abs(want[rid.rstrip("x")]).max(), f"{rid} position {pos} (graphs={graphs})"
            assert len(got) == sum(len(v) for v in reqs.values())
    finally:
        unregister_architecture("ToyParallelForCausalLM")
        unregister_part("norm", "toy_centered")
        unregister_part("block", "toy_parallel")


def test_norms_and_activation_folded_into_the_products_change_nothing_but_rounding(tmp_path, monkeypatch):
    """Steps of few tokens fold the norms, the residual sums and the SwiGLU activation into the
    epilogues of the engine's own GEMM (widths that are multiples of 64 allow it).  The same
    trace with the folding switched off, and the float32 path, must give the same logits up to
    bfloat16 rounding; and the folded path must really have run."""
    from tests.tiny_configs import TINY_A, tiny_weights, write_model_folder
    from tokensprint_b200 import ops
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.parts import linear as linear_module

    cfg = dict(TINY_A)
    cfg.update(hidden_size=192, intermediate_size=320, num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_hidden_layers=3,
               vocab_size=520, tie_word_embeddings=False)
    weights = tiny_weights(cfg, 5, std=0.05)
    folder = write_model_folder(tmp_path / "m", cfg, weights)
    g = torch.Generator().manual_seed(1)
    requests = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate((40, 9, 77))}
    steps = trace_decode_tail(requests, 24)

    calls = []
    real = ops.gemm_skinny_fused
    monkeypatch.setattr(ops, "gemm_skinny_fused", lambda *a, **k: (calls.append(k.get("mode", 0)), real(*a, **k))[1])
    folded = replay_in_process(TraceReplayer.from_folder(folder, "bfloat16", 512), steps)
    assert {0, ops.GEMM_EPILOGUE_SWIGLU, ops.GEMM_EPILOGUE_RESIDUAL_NORM} <= set(calls), "the folded path did not run"
    calls.clear()
    monkeypatch.setattr(linear_module, "FOLD_NORMS", False)
    plain_path = replay_in_process(TraceReplayer.from_folder(folder, "bfloat16", 512), steps)
    assert not calls
    exact = replay_in_process(TraceReplayer.from_folder(folder, "float32", 512), steps)
    scale = max(float(abs(v).max()) for v in exact.values())
    assert set(folded) == set(plain_path) == set(exact)
    for key in exact:
        assert float(abs(folded[key] - exact[key]).max()) < 4e-2 * scale, f"folded, {key}"
        assert float(abs(plain_path[key] - exact[key]).max()) < 4e-2 * scale, f"unfolded, {key}"
    # the folded path rounds less often than the unfolded one: on average it is no further from float32
    err_f = sum(float(abs(folded[k] - exact[k]).mean()) for k in exact)
    err_u = sum(float(abs(plain_path[k] - exact[k]).mean()) for k in exact)
    assert err_f < 1.5 * err_u


# ---------------------------------------------------------------------------
# a third toy architecture: what happens outside the layers (an embedding multiplier, a soft cap
# and a bias on the logits) and a mixer whose cache rows are not attention's (keys wider than
# values, one head) - all defined here


@dataclass(frozen=True)
class ToyWideKeyConfig:
    vocab_size: int = 83
    hidden_size: int = 40
    num_hidden_layers: int = 2
    key_size: int = 24
    value_size: int = 8
    intermediate_size: int = 56
    embedding_multiplier: float = 3.5
    logit_cap: float = 4.0
    rms_norm_eps: float = 1e-6
    architectures: tuple = ("ToyWideKeyForCausalLM",)

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        return d

    def save(self, folder):
        import json
        from pathlib import Path

        Path(folder).mkdir(parents=True, exist_ok=True)
        (Path(folder) / "config.json").write_text(json.dumps(self.to_dict()))


def _register_wide_key_toy():
    from tokensprint_b200.config.registry import register_architecture
    from tokensprint_b200.models.spec import ModelSpec
    from tokensprint_b200.parts.base import CacheNeed, Mixer, PartSpec, TensorSpec, Transform, register_part

    @register_part("transform", "toy_multiplier", replace=True)
    class Multiplier(Transform):
        graph_safe = True

        def __init__(self, bctx, *, factor):
            self.factor = float(factor)

        def forward(self, x, step):
            return x.mul_(self.factor)

    @register_part("transform", "toy_cap_and_bias", replace=True)
    class CapAndBias(Transform):
        """logits -> cap * tanh(logits / cap) + bias, the bias a tensor of the checkpoint."""

        graph_safe = True

        def __init__(self, bctx, *, cap, bias, size):
            self.cap, self.bias_name, self.size = float(cap), bias, size

        def tensor_specs(self):
            return [TensorSpec(self.bias_name, (self.size,), "vector")]

        def load(self, tensors):
            self.bias = tensors[self.bias_name]

        def forward(self, x, step):
            return torch.tanh(x / self.cap) * self.cap + self.bias

    @register_part("mixer", "toy_wide_keys", replace=True)
    class WideKeyMixer(Mixer):
        """One head, keys of `key_size` and values of `value_size` entries, both paged: the two
        pools of its cache have different row shapes.  Plain torch on the pages and tables it is
        handed; the host's copies of the step's lengths say which rows belong to whom."""

        def __init__(self, bctx, *, hidden_size, key_size, value_size, prefix):
            self.H, self.dk, self.dv, self.prefix = hidden_size, key_size, value_size, prefix

        def cache_need(self):
            return CacheNeed(kind="full", k_row=(self.dk,), v_row=(self.dv,))

        def tensor_specs(self):
            p = self.prefix
            return [TensorSpec(p + "q", (self.dk, self.H)), TensorSpec(p + "k", (self.dk, self.H)),
                    TensorSpec(p + "v", (self.dv, self.H)), TensorSpec(p + "o", (self.H, self.dv))]

        def load(self, tensors):
            self.w = {n: tensors[self.prefix + n] for n in "qkvo"}

        def forward(self, x, step, cache):
            P = step.page_size
            assert cache.k_pages.shape[1:] == (P, self.dk) and cache.v_pages.shape[1:] == (P, self.dv)
            tables = step.groups[cache.group]
            q, k, v = x @ self.w["q"].t(), x @ self.w["k"].t(), x @ self.w["v"].t()
            k_flat, v_flat = cache.k_pages.view(-1, self.dk), cache.v_pages.view(-1, self.dv)
            slots = tables.slot_mapping[: x.shape[0]].long()
            k_flat[slots] = k
            v_flat[slots] = v
            out = torch.empty((x.shape[0], self.dv), device=x.device, dtype=x.dtype)
            t0 = 0
            for b, (start, n) in enumerate(zip(step.host_seq_starts, step.host_seq_lens)):
                pos = torch.arange(start + n, device=x.device)
                held = tables.block_table[b].long()[pos // P] * P + pos % P
                scores = (q[t0 : t0 + n] @ k_flat[held].t()) * self.dk**-0.5
                hidden_keys = pos[None, :] > (start + torch.arange(n, device=x.device))[:, None]
                out[t0 : t0 + n] = torch.softmax(scores.masked_fill(hidden_keys, float("-inf")), dim=-1) @ v_flat[held]
                t0 += n
            return out @ self.w["o"].t()

    @register_architecture("ToyWideKeyForCausalLM", config_from_dict=lambda d: ToyWideKeyConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items()}))
    def build(cfg: ToyWideKeyConfig):
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"w.{i}."
            norm = {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps}
            layers.append(PartSpec("pre_norm", {
                "mixer": PartSpec("toy_wide_keys", {"hidden_size": cfg.hidden_size, "key_size": cfg.key_size, "value_size": cfg.value_size, "prefix": p + "mix."}),
                "feed_forward": PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                                                    "gate": p + "gate", "up": p + "up", "down": p + "down"}),
                "mixer_norm": PartSpec("rmsnorm", {**norm, "weight": p + "n1"}),
                "ffn_norm": PartSpec("rmsnorm", {**norm, "weight": p + "n2"})}))
        return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, embedding="w.embed", layers=layers,
                         final_norm=PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps, "weight": "w.norm"}),
                         lm_head=None, max_positions=512,
                         embedding_transform=PartSpec("toy_multiplier", {"factor": cfg.embedding_multiplier}),
                         logits_transform=PartSpec("toy_cap_and_bias", {"cap": cfg.logit_cap, "bias": "w.logit_bias", "size": cfg.vocab_size}))


def _plain_wide_key_toy(weights, cfg: ToyWideKeyConfig, ids):
    w = {k: v.double() for k, v in weights.items()}
    T = len(ids)
    h = plain.embedding(w["w.embed"], ids) * cfg.embedding_multiplier
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    for i in range(cfg.num_hidden_layers):
        p = f"w.{i}."
        x = plain.rms_norm(h, w[p + "n1"], cfg.rms_norm_eps)
        q, k, v = x @ w[p + "mix.q"].T, x @ w[p + "mix.k"].T, x @ w[p + "mix.v"].T
        scores = (q @ k.T * cfg.key_size**-0.5).masked_fill(~causal, float("-inf"))
        h = h + (torch.softmax(scores, dim=-1) @ v) @ w[p + "mix.o"].T
        x = plain.rms_norm(h, w[p + "n2"], cfg.rms_norm_eps)
        g, u = x @ w[p + "gate"].T, x @ w[p + "up"].T
        h = h + (g * torch.sigmoid(g) * u) @ w[p + "down"].T
    logits = plain.rms_norm(h, w["w.norm"], cfg.rms_norm_eps) @ w["w.embed"].T
    return torch.tanh(logits / cfg.logit_cap) * cfg.logit_cap + w["w.logit_bias"]


def test_a_toy_model_with_transforms_outside_the_layers_and_keys_wider_than_values(tmp_path):
    """An embedding multiplier, a soft cap and a bias on the logits, and a cache whose two pools
    have different row shapes: registered here, built from config.json, stepped in all four
    cuttings with pages used again, without a change to the framework's files."""
    from tokensprint_b200.config.registry import unregister_architecture
    from tokensprint_b200.engine.replay import TraceReplayer
    from tokensprint_b200.parts.base import unregister_part
    from tokensprint_b200.weights.loader import write_random_model
    from tokensprint_b200.weights.safetensors_io import SafetensorsFolder

    _register_wide_key_toy()
    try:
        cfg = ToyWideKeyConfig()
        folder = write_random_model(tmp_path / "wide", cfg, seed=13, dtype="float32", std=0.2)
        files = SafetensorsFolder(folder)
        weights = {n: files.tensor(n).clone() for n in files.keys()}
        assert weights["w.0.mix.k"].shape == (24, 40) and weights["w.0.mix.v"].shape == (8, 40) and "w.logit_bias" in weights
        g = torch.Generator().manual_seed(9)
        requests = {f"r{i}": torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((2, 19, 40, 66))}
        want = {rid: _plain_wide_key_toy(weights, cfg, ids) for rid, ids in requests.items()}
        assert max(float(v.abs().max()) for v in want.values()) > 0.8 * cfg.logit_cap, "the cap is not exercised"
        many = dict(requests)
        many.update({k + "x": v for k, v in requests.items()})
        for steps, reqs in ((trace_whole(requests), requests), (trace_decode_tail(requests, 16), requests),
                            (trace_portions(requests), requests), (trace_mixed(many, 256, seed=4), many)):
            replayer = TraceReplayer.from_folder(folder, "float32", 256, max_live=4)
            replayer.runner.poison_freed_pages = True
            tensors = replayer.runner.cache_tensors
            assert tensors.k[0].shape[2:] == (24,) and tensors.v[0].shape[2:] == (8,)
            assert replayer.runner.page_bytes == [2 * 16 * (24 + 8) * 4]
            got = replay_in_process(replayer, steps)
            for (rid, pos), row in got.items():
                ref = want[rid.rstrip("x")][pos].numpy()
                assert abs(row - ref).max() < 1e-4 * abs(want[rid.rstrip("x")]).max(), f"{rid} position {pos}"
            assert len(got) == sum(len(v) for v in reqs.values())
    finally:
        unregister_architecture("ToyWideKeyForCausalLM")
        for category, name in (("mixer", "toy_wide_keys"), ("transform", "toy_multiplier"), ("transform", "toy_cap_and_bias")):
            unregister_part(category, name)


def test_cache_size_comes_from_free_memory_when_no_page_count_is_given(tmp_path):
    """A runner built without a page count measures a step of the largest size, sizes its pool from
    what is free after it, and generates with it."""
    from tests.tiny_configs import TINY_B, tiny_weights, write_model_folder
    from tokensprint_b200.config.engine_config import Config, SamplingParams
    from tokensprint_b200.engine.llm_engine import LLMEngine
    from tokensprint_b200.models.api import load_model

    folder = write_model_folder(tmp_path / "m", TINY_B, tiny_weights(TINY_B, 3, std=0.05))
    model, _ = load_model(folder, device=DEV, dtype="bfloat16")
    torch.cuda.synchronize()
    free_before, total = torch.cuda.mem_get_info()
    utilization = 0.05  # a small share: the test must not take the GPU's memory from whoever runs beside it
    engine = LLMEngine(model, Config(model=str(folder), max_model_len=256, max_num_batched_tokens=512, max_num_seqs=8,
                                     kvcache_block_size=16, num_kvcache_blocks=-1, gpu_memory_utilization=utilization, dtype="bfloat16"))
    runner = engine.model_runner
    s = runner.sizing
    assert s is not None and s["pages"] == runner.num_pages[0] == engine.config.num_kvcache_blocks
    assert s["step_tokens"] == 512 and s["step_peak_bytes"] > 512 * TINY_B["hidden_size"] * 4  # at least the residual stream
    assert s["bytes_per_page"] == 2 * 16 * TINY_B["num_key_value_heads"] * TINY_B["head_dim"] * 2 * TINY_B["num_hidden_layers"]
    pool_bytes = s["pages"] * s["bytes_per_page"]
    budget = s["free_bytes"] * utilization - s["step_peak_bytes"] - s["graph_reserve_bytes"] - s["margin_bytes"]
    assert 0 <= budget - pool_bytes < s["bytes_per_page"], "the pool is what the budget allows, to the page"
    assert pool_bytes < free_before * utilization
    assert s["graph_reserve_bytes"] > 0  # graphs are on by default and keep their logits
    out = engine.generate([[1, 2, 3, 4, 5], list(range(10, 60))], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), use_tqdm=False)
    assert [len(o) for o in out] == [6, 6]
    assert runner.cache_manager.pages_in_use() == 0

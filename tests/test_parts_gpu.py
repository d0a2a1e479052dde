"""Each kind of part alone, and models put together from parts in ways the built-in architecture does not use:
a windowed attention with partial rotary width and no q/k norm, a layer that runs twice with the second run
reading the first run's cache, and a toy mixer with per-request state that is defined here, registered, built and
stepped without touching the framework's files; likewise a toy feed-forward with a router and experts and a toy
position encoding.  All are replayed whole, in portions and mixed, and compared
with plain restatements written in this file from ``plain_qwen3``'s functions.
"""
from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import traces
from conftest import TOLERANCE, random_tokens

pytestmark = pytest.mark.gpu

H, V, MAXPOS = 48, 211, 400


def _register(name, spec_fn):
    from cuinfer_b200.config import register_architecture
    register_architecture(name, lambda raw: SimpleNamespace(**raw), spec_fn, replace=True)


def _base_cfg(name, **kw):
    return dict(architectures=[name], hidden_size=H, vocab_size=V, max_position_embeddings=MAXPOS, **kw)


def _model_spec(cfg, layers, **kw):
    from cuinfer_b200.parts import ModelSpec, PartSpec
    return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
                     layers=tuple(layers), final_norm=PartSpec("rmsnorm", eps=cfg.eps), lm_head_name="lm_head.weight", **kw)


def _replay_all(folder, dtype, requests, tmp_path, plain_fn, block=16):
    """whole / tail / portions / mixed with page reuse, each against ``plain_fn(ids) -> logits``."""
    worst = 0.0
    for label, steps in [("whole", traces.whole(requests)), ("tail", traces.tail_decode(requests, 20)),
                         ("portions", traces.portions(requests)), ("mixed", traces.mixed(requests, max_live=3))]:
        out = str(tmp_path / f"{label}_{dtype}")
        traces.replay_in_process(folder, dtype, steps, out, traces.live_token_peak(steps), block)
        got = traces.collect(steps, out, V)
        for rid, toks in requests.items():
            ref = plain_fn(list(toks)).numpy()
            scale = float(np.abs(ref).max())
            for pos, row in sorted(got[rid].items()):
                err = float(np.abs(row - ref[pos]).max()) / scale
                worst = max(worst, err)
                assert err <= TOLERANCE[dtype], f"{label}: request {rid} first wrong position {pos} (error {err:.3e})"
    from conftest import note_error
    note_error(dtype, "toy parts", worst)
    return worst


# ---- 1. windowed attention, partial rotary width, no q/k norm, custom scale ------------------------------------

WINDOW, ROT, NQ, NKV, D, SCALE = 21, 8, 4, 2, 24, 0.31


def _window_spec(cfg):
    from cuinfer_b200.parts import LayerSpec, PartSpec
    pos = PartSpec("rope_neox", theta=cfg.theta, rotary_dim=ROT, max_positions=cfg.max_position_embeddings)
    mixer = PartSpec("attention", name="attn", num_heads=NQ, num_kv_heads=NKV, head_dim=D, qk_norm=False,
                     scale=SCALE, window=WINDOW, position=pos)
    layer = lambda i: LayerSpec(prefix=f"blk.{i}", block=PartSpec("prenorm", norm_names=("n1", "n2")), mixer=mixer,
                                feed_forward=PartSpec("swiglu", name="ff", intermediate_size=72),
                                norm=PartSpec("rmsnorm", eps=cfg.eps))
    return _model_spec(cfg, [layer(0), layer(1)])


def _window_plain(cfg, w, ids):
    x = P.embed(w["model.embed_tokens.weight"], ids)
    n = len(ids)
    pos = torch.arange(n)
    cos, sin = P.rope_cos_sin(cfg["theta"], ROT, pos)
    for i in range(2):
        p = f"blk.{i}"
        h = P.rms_norm(x, w[f"{p}.n1.weight"], cfg["eps"])
        q = P.apply_rope((h @ w[f"{p}.attn.q_proj.weight"].T).view(n, NQ, D), cos, sin)
        k = P.apply_rope((h @ w[f"{p}.attn.k_proj.weight"].T).view(n, NKV, D), cos, sin)
        v = (h @ w[f"{p}.attn.v_proj.weight"].T).view(n, NKV, D)
        x = x + P.causal_attention(q, k, v, SCALE, WINDOW).reshape(n, -1) @ w[f"{p}.attn.o_proj.weight"].T
        x = x + P.swiglu(P.rms_norm(x, w[f"{p}.n2.weight"], cfg["eps"]), w, f"{p}.ff")
    return P.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_attention_with_partial_rotary(dtype, tmp_path):
    from cuinfer_b200.engine import replay
    from cuinfer_b200.weights import write_random_model

    _register("ToyWindowLM", _window_spec)
    cfg = _base_cfg("ToyWindowLM", theta=5000.0, eps=1e-5)
    folder = write_random_model(str(tmp_path / "m"), cfg, 3, std=0.08 if dtype == "float32" else 0.05, gain_std=0.1,
                                dtype=dtype)
    pcfg, w = P.load_folder(folder)
    requests = {f"r{i}": random_tokens(V, n, 300 + i) for i, n in enumerate([70, 45, 100, 33])}
    _replay_all(folder, dtype, requests, tmp_path, lambda ids: _window_plain(pcfg, w, ids))
    # the windowed group gives pages back while a request is still running
    runner = replay.make_runner(folder, dtype, 256, 16)
    assert runner.groups[0].window == WINDOW
    runner.reserve("a", 100)
    from cuinfer_b200.engine import StepEntry
    runner.step([StepEntry("a", requests["r2"], [99])])
    table = runner.manager.block_table("a", 0)
    assert table[0] == -1 and table[3] == -1 and table[-1] >= 0 and sum(p >= 0 for p in table) <= 3


# ---- 2. one layer run twice; the second run reads the first run's cache ------------------------------------------

def _twice_spec(cfg):
    from cuinfer_b200.parts import LayerSpec, PartSpec
    pos = PartSpec("rope_neox", theta=cfg.theta, rotary_dim=16, max_positions=cfg.max_position_embeddings)
    mixer = PartSpec("attention", name="attn", num_heads=3, num_kv_heads=1, head_dim=16, qk_norm=True,
                     qk_norm_eps=cfg.eps, position=pos)
    layer = LayerSpec(prefix="blk.0", block=PartSpec("prenorm", norm_names=("n1", "n2")), mixer=mixer,
                      feed_forward=PartSpec("swiglu", name="ff", intermediate_size=40), norm=PartSpec("rmsnorm", eps=cfg.eps))
    return _model_spec(cfg, [layer], order=(0, 0), cache_source={1: 0})


def _twice_plain(cfg, w, ids):
    x = P.embed(w["model.embed_tokens.weight"], ids)
    n = len(ids)
    cos, sin = P.rope_cos_sin(cfg["theta"], 16, torch.arange(n))
    p = "blk.0"
    kept = None
    for run in range(2):
        h = P.rms_norm(x, w[f"{p}.n1.weight"], cfg["eps"])
        q = (h @ w[f"{p}.attn.q_proj.weight"].T).view(n, 3, 16)
        q = P.apply_rope(P.rms_norm(q, w[f"{p}.attn.q_norm.weight"], cfg["eps"]), cos, sin)
        if run == 0:
            k = (h @ w[f"{p}.attn.k_proj.weight"].T).view(n, 1, 16)
            k = P.apply_rope(P.rms_norm(k, w[f"{p}.attn.k_norm.weight"], cfg["eps"]), cos, sin)
            v = (h @ w[f"{p}.attn.v_proj.weight"].T).view(n, 1, 16)
            kept = (k, v)
        k, v = kept                                   # the second run attends over the first run's keys and values
        x = x + P.causal_attention(q, k, v, 0.25).reshape(n, -1) @ w[f"{p}.attn.o_proj.weight"].T
        x = x + P.swiglu(P.rms_norm(x, w[f"{p}.n2.weight"], cfg["eps"]), w, f"{p}.ff")
    return P.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_run_twice_sharing_a_cache(dtype, tmp_path):
    from cuinfer_b200.engine import replay
    from cuinfer_b200.weights import write_random_model

    _register("ToyTwiceLM", _twice_spec)
    cfg = _base_cfg("ToyTwiceLM", theta=10000.0, eps=1e-6)
    folder = write_random_model(str(tmp_path / "m"), cfg, 4, std=0.08 if dtype == "float32" else 0.05, dtype=dtype)
    pcfg, w = P.load_folder(folder)
    requests = {f"r{i}": random_tokens(V, n, 400 + i) for i, n in enumerate([50, 81, 37])}
    _replay_all(folder, dtype, requests, tmp_path, lambda ids: _twice_plain(pcfg, w, ids))
    runner = replay.make_runner(folder, dtype, 64, 16)
    assert len(runner.groups) == 1 and runner.groups[0].runs == (0,)          # one cache for two runs
    assert [t.name for t in runner.model.tensors()].count("blk.0.attn.q_proj.weight") == 1


# ---- 3. a toy mixer with state of its own ---------------------------------------------------------------------------

def _define_toy_mixer():
    from cuinfer_b200.parts import MIXERS, Mixer, StateNeed, TensorSpec

    if "running_mean" in MIXERS:
        return

    @MIXERS.register("running_mean")
    class RunningMean(Mixer):
        """y_t = W · mean(x_0 .. x_t).  Per-request state: the running sum of x and the count, 32-bit."""

        capturable = False      # loops over the batch's state slots on the host: never replayed from a CUDA graph

        def tensors(self):
            return [TensorSpec(f"{self.prefix}.proj.weight", (self.hidden_size, self.hidden_size))]

        def load(self, store):
            self.weight = store.get(self.tensors()[0]).float()

        def state_need(self):
            return StateNeed((self.hidden_size + 1,), "float32")

        def forward(self, x, ctx, run):
            state = ctx.run_state(run)
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            starts = ctx.query_start_loc_host
            for r, slot in enumerate(ctx.state_slots_host):
                rows = x[starts[r]:starts[r + 1]].float()
                sums = torch.cumsum(rows, 0) + state[slot, :-1]
                counts = state[slot, -1] + torch.arange(1, rows.shape[0] + 1, device=x.device, dtype=torch.float32)
                out[starts[r]:starts[r + 1]] = sums / counts[:, None]
                state[slot, :-1] = sums[-1]
                state[slot, -1] = counts[-1]
            return (out @ self.weight.T).to(x.dtype)


def _toy_spec(cfg):
    from cuinfer_b200.parts import LayerSpec, PartSpec
    _define_toy_mixer()
    pos = PartSpec("rope_neox", theta=cfg.theta, rotary_dim=16, max_positions=cfg.max_position_embeddings)
    attn = PartSpec("attention", name="attn", num_heads=2, num_kv_heads=2, head_dim=16, qk_norm=True, qk_norm_eps=cfg.eps,
                    position=pos)
    block = PartSpec("prenorm", norm_names=("n1", "n2"))
    ff = PartSpec("swiglu", name="ff", intermediate_size=56)
    norm = PartSpec("rmsnorm", eps=cfg.eps)
    return _model_spec(cfg, [
        LayerSpec("blk.0", block, PartSpec("running_mean", name="mean"), ff, norm),      # state, no pages
        LayerSpec("blk.1", block, attn, ff, norm),                                       # pages, no state
        LayerSpec("blk.2", block, PartSpec("running_mean", name="mean"), ff, norm),
    ])


def _toy_plain(cfg, w, ids):
    x = P.embed(w["model.embed_tokens.weight"], ids)
    n = len(ids)
    cos, sin = P.rope_cos_sin(cfg["theta"], 16, torch.arange(n))
    for i in range(3):
        p = f"blk.{i}"
        h = P.rms_norm(x, w[f"{p}.n1.weight"], cfg["eps"])
        if i != 1:
            mean = torch.cumsum(h, 0) / torch.arange(1, n + 1, dtype=torch.float32)[:, None]
            x = x + mean @ w[f"{p}.mean.proj.weight"].T
        else:
            q = (h @ w[f"{p}.attn.q_proj.weight"].T).view(n, 2, 16)
            k = (h @ w[f"{p}.attn.k_proj.weight"].T).view(n, 2, 16)
            v = (h @ w[f"{p}.attn.v_proj.weight"].T).view(n, 2, 16)
            q = P.apply_rope(P.rms_norm(q, w[f"{p}.attn.q_norm.weight"], cfg["eps"]), cos, sin)
            k = P.apply_rope(P.rms_norm(k, w[f"{p}.attn.k_norm.weight"], cfg["eps"]), cos, sin)
            x = x + P.causal_attention(q, k, v, 0.25).reshape(n, -1) @ w[f"{p}.attn.o_proj.weight"].T
        x = x + P.swiglu(P.rms_norm(x, w[f"{p}.n2.weight"], cfg["eps"]), w, f"{p}.ff")
    return P.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype, tmp_path):
    from cuinfer_b200.engine import replay
    from cuinfer_b200.weights import write_random_model

    _register("ToyStateLM", _toy_spec)
    cfg = _base_cfg("ToyStateLM", theta=10000.0, eps=1e-6)
    folder = write_random_model(str(tmp_path / "m"), cfg, 5, std=0.08 if dtype == "float32" else 0.05, dtype=dtype)
    pcfg, w = P.load_folder(folder)
    # more requests than live slots, so that state slots are used again and must start from zero
    requests = {f"r{i}": random_tokens(V, n, 500 + i) for i, n in enumerate([40, 23, 66, 31, 52])}
    _replay_all(folder, dtype, requests, tmp_path, lambda ids: _toy_plain(pcfg, w, ids))
    runner = replay.make_runner(folder, dtype, 128, 16)
    assert sorted(runner.storage.state) == [0, 2] and runner.storage.state[0].shape == (8, H + 1)
    assert [g.runs for g in runner.groups] == [(1,)]


# ---- 4. a toy feed-forward with routing and a toy position encoding ---------------------------------------------------

EXPERTS, TOPK, EXPERT_WIDTH, STRETCH = 5, 2, 24, 3.5


def _define_toy_routed_parts():
    from cuinfer_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding, TensorSpec

    if "toy_routed" not in FEED_FORWARDS:
        @FEED_FORWARDS.register("toy_routed")
        class ToyRouted(FeedForward):
            """y = sum over a token's top-k experts of softmax-weight x relu(x W_in^T) W_out^T; router in 32 bits."""

            capturable = False      # sizes its expert products from the routing (torch.nonzero waits for the device)

            def tensors(self):
                e, w, h = self.spec.experts, self.spec.width, self.hidden_size
                return [TensorSpec(f"{self.prefix}.router.weight", (e, h)),
                        TensorSpec(f"{self.prefix}.w_in", (e, w, h)), TensorSpec(f"{self.prefix}.w_out", (e, h, w))]

            def load(self, store):
                self.router, self.w_in, self.w_out = (store.get(t) for t in self.tensors())

            def forward(self, x, ctx):
                logits = x.float() @ self.router.float().T
                top, idx = torch.topk(logits, self.spec.top_k, dim=-1)
                weight = torch.softmax(top, dim=-1)
                out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
                for e in range(self.spec.experts):
                    rows, slot = torch.nonzero(idx == e, as_tuple=True)
                    if rows.numel():
                        hidden = torch.relu(x[rows] @ self.w_in[e].T)
                        out.index_add_(0, rows, (hidden @ self.w_out[e].T).float() * weight[rows, slot][:, None])
                return out.to(x.dtype)

    if "toy_stretched" not in POSITION_ENCODINGS:
        @POSITION_ENCODINGS.register("toy_stretched")
        class ToyStretched(PositionEncoding):
            """Rotary angles (p / stretch) / (1 + i): another law of frequencies, same table shape."""

            def __init__(self, spec, **kw):
                super().__init__(spec, **kw)
                self.rotary_dim = int(spec.rotary_dim)
                self._device, self._table = None, None

            def load(self, store):
                self._device = store.device

            def table(self):
                if self._table is None:
                    self._table = _stretched_table(self.spec.max_positions, self.rotary_dim, self.spec.stretch).to(self._device)
                return self._table


def _stretched_table(positions, rotary_dim, stretch):
    pos = torch.arange(positions, dtype=torch.float32) / float(stretch)
    freq = 1.0 / (1.0 + torch.arange(rotary_dim // 2, dtype=torch.float32))
    angle = pos[:, None] * freq[None, :]
    return torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1).contiguous()


def _routed_spec(cfg):
    from cuinfer_b200.parts import LayerSpec, PartSpec
    _define_toy_routed_parts()
    pos = PartSpec("toy_stretched", rotary_dim=12, max_positions=cfg.max_position_embeddings, stretch=STRETCH)
    attn = PartSpec("attention", name="attn", num_heads=4, num_kv_heads=1, head_dim=16, qk_norm=False, position=pos)
    block = PartSpec("prenorm", norm_names=("n1", "n2"))
    routed = PartSpec("toy_routed", name="moe", experts=EXPERTS, top_k=TOPK, width=EXPERT_WIDTH)
    norm = PartSpec("rmsnorm", eps=cfg.eps)
    return _model_spec(cfg, [
        LayerSpec("blk.0", block, attn, routed, norm),                                           # experts
        LayerSpec("blk.1", block, attn, PartSpec("swiglu", name="ff", intermediate_size=40), norm),   # dense
        LayerSpec("blk.2", block, attn, routed, norm),
    ])


def _routed_plain(cfg, w, ids, gaps=None):
    x = P.embed(w["model.embed_tokens.weight"], ids)
    n = len(ids)
    table = _stretched_table(cfg["max_position_embeddings"], 12, STRETCH)[:n]
    cos, sin = table[..., 0], table[..., 1]
    for i in range(3):
        p = f"blk.{i}"
        h = P.rms_norm(x, w[f"{p}.n1.weight"], cfg["eps"])
        q = P.apply_rope((h @ w[f"{p}.attn.q_proj.weight"].T).view(n, 4, 16), cos, sin)
        k = P.apply_rope((h @ w[f"{p}.attn.k_proj.weight"].T).view(n, 1, 16), cos, sin)
        v = (h @ w[f"{p}.attn.v_proj.weight"].T).view(n, 1, 16)
        x = x + P.causal_attention(q, k, v, 0.25).reshape(n, -1) @ w[f"{p}.attn.o_proj.weight"].T
        h = P.rms_norm(x, w[f"{p}.n2.weight"], cfg["eps"])
        if i == 1:
            x = x + P.swiglu(h, w, f"{p}.ff")
            continue
        logits = h @ w[f"{p}.moe.router.weight"].T
        if gaps is not None:
            ordered = torch.sort(logits, dim=-1, descending=True).values
            gaps.append(float(((ordered[:, TOPK - 1] - ordered[:, TOPK]) / (ordered[:, 0] - ordered[:, -1])).min()))
        for t in range(n):
            top, idx = torch.topk(logits[t], TOPK)
            weight = torch.softmax(top, dim=-1)
            for c in range(TOPK):
                e = int(idx[c])
                x[t] += weight[c] * (torch.relu(h[t] @ w[f"{p}.moe.w_in"][e].T) @ w[f"{p}.moe.w_out"][e].T)
    return P.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_toy_position_encoding(dtype, tmp_path):
    """A feed-forward with a router and experts, and a position encoding with another law of angles, both defined
    here: registered, chosen layer by layer beside the dense feed-forward, built, loaded by tensor name and stepped."""
    from cuinfer_b200.engine import replay
    from cuinfer_b200.weights import write_random_model

    _register("ToyRoutedLM", _routed_spec)
    cfg = _base_cfg("ToyRoutedLM", eps=3e-6)
    folder = write_random_model(str(tmp_path / "m"), cfg, 6, std=0.08 if dtype == "float32" else 0.05, dtype=dtype)
    pcfg, w = P.load_folder(folder)
    requests = {f"r{i}": random_tokens(V, n, 600 + i) for i, n in enumerate([48, 27, 70])}
    if dtype == "bfloat16":
        # bfloat16 rounding may turn a near-tie between two experts the other way, and every later position then
        # differs; so the bfloat16 runs take token sequences whose router logits have a clear margin at every token
        requests, seed = {}, 700
        while len(requests) < 3 and seed < 900:
            toks = random_tokens(V, 22 + seed % 9, seed)
            if _routing_margin(pcfg, w, toks) > 0.01:
                requests[f"r{seed}"] = toks
            seed += 1
        assert len(requests) == 3, "too few token sequences with a clear routing margin"
    _replay_all(folder, dtype, requests, tmp_path, lambda ids: _routed_plain(pcfg, w, ids))
    runner = replay.make_runner(folder, dtype, 128, 16)
    names = [t.name for t in runner.model.tensors()]
    assert "blk.0.moe.router.weight" in names and "blk.1.ff.down_proj.weight" in names and "blk.2.moe.w_out" in names
    assert type(runner.model.blocks[0].feed_forward).__name__ == "ToyRouted"
    assert type(runner.model.blocks[0].mixer.position).__name__ == "ToyStretched"


def _routing_margin(cfg, w, ids):
    """Smallest gap between the k-th and (k+1)-th router logit over the tokens and routed layers, relative to the
    logits' spread, along the plain forward pass."""
    gaps = []
    _routed_plain(cfg, w, ids, gaps)
    return min(gaps)


# ---- 4b. the toy architectures through the entry point, with the engine's default settings --------------------------

def _plain_greedy(plain_fn, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(plain_fn(ids)[-1])))
    return ids[len(prompt):]


@pytest.mark.parametrize("arch", ["window", "twice", "state", "routed"])
def test_toy_architectures_generate_with_default_settings(arch, tmp_path):
    """``LLM.generate`` with CUDA graphs and run-ahead on (the defaults) on models made of other parts: the windowed
    and the cache-sharing attention are replayed from decode graphs; the toy mixer with state and the routed toy
    feed-forward say ``capturable = False`` and the engine runs their steps eagerly, host arrays filled in.  Greedy
    float32 tokens equal the plain restatement's in every case."""
    from cuinfer_b200 import LLM, SamplingParams
    from cuinfer_b200.weights import write_random_model

    name, spec_fn, plain, extra = {
        "window": ("ToyWindowLM", _window_spec, _window_plain, dict(theta=5000.0, eps=1e-5)),
        "twice": ("ToyTwiceLM", _twice_spec, _twice_plain, dict(theta=10000.0, eps=1e-6)),
        "state": ("ToyStateLM", _toy_spec, _toy_plain, dict(theta=10000.0, eps=1e-6)),
        "routed": ("ToyRoutedLM", _routed_spec, _routed_plain, dict(eps=3e-6)),
    }[arch]
    _register(name, spec_fn)
    cfg = _base_cfg(name, **extra)
    folder = write_random_model(str(tmp_path / "m"), cfg, 11, std=0.08, gain_std=0.1, dtype="float32")
    pcfg, w = P.load_folder(folder)
    prompts = [random_tokens(V, n, 800 + i) for i, n in enumerate([30, 7, 52, 19, 3])]
    llm = LLM(folder, dtype="float32", num_blocks=48, max_num_seqs=8)          # everything else as it comes
    assert llm.config.enable_cuda_graph and llm.config.decode_run_ahead
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=26, ignore_eos=True))
    for prompt, res in zip(prompts, out):
        assert res.token_ids == _plain_greedy(lambda ids: plain(pcfg, w, ids), prompt, 26), (arch, len(prompt))
    runner = llm.engine.runner
    capturable = arch in ("window", "twice")
    assert runner.model.capturable == capturable
    assert (runner.graph_steps > 20) == capturable          # graphs where the parts allow them, eager steps elsewhere
    runner.manager.check()
    assert not runner.manager.live_requests()


# ---- 5. single parts against their formulas ---------------------------------------------------------------------------

class DictStore:
    def __init__(self, tensors, device="cuda:0"):
        self.tensors, self.device = tensors, torch.device(device)

    def get(self, spec):
        return self.tensors[spec.name].to(self.device)

    def get_stacked(self, specs):
        return torch.cat([self.get(s) for s in specs], 0).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_feed_forward_and_position_parts_alone(dtype):
    from cuinfer_b200.parts import FEED_FORWARDS, NORMS, POSITION_ENCODINGS, PartSpec, ResidualStream

    g = torch.Generator().manual_seed(7)
    hid, inter, rows = 88, 136, 9
    tol = 2e-6 if dtype == torch.float32 else 1.5e-2
    # norm: folds the pending delta into the residual, then normalises
    norm = NORMS.get("rmsnorm")(PartSpec("rmsnorm", eps=2e-5), hidden_size=hid, prefix="n", dtype=dtype)
    assert [(t.name, t.shape, t.init) for t in norm.tensors()] == [("n.weight", (hid,), "ones")]
    gain = 1 + 0.2 * torch.randn(hid, generator=g)
    norm.load(DictStore({"n.weight": gain}))
    res, delta = torch.randn(rows, hid, generator=g), torch.randn(rows, hid, generator=g).to(dtype)
    stream = ResidualStream(res.clone().cuda(), delta.cuda())
    out = norm.add_norm(stream)
    assert stream.pending is None and out.dtype == dtype
    want_res = res + delta.float()
    assert float((stream.residual.cpu() - want_res).abs().max()) < 1e-6
    want = P.rms_norm(want_res, gain, 2e-5)
    assert float((out.float().cpu() - want).abs().max()) / float(want.abs().max()) < tol
    # feed-forward
    ff = FEED_FORWARDS.get("swiglu")(PartSpec("swiglu", intermediate_size=inter), hidden_size=hid, prefix="ff", dtype=dtype)
    assert sorted(t.name for t in ff.tensors()) == ["ff.down_proj.weight", "ff.gate_proj.weight", "ff.up_proj.weight"]
    wts = {n: (0.2 * torch.randn(s, generator=g)).to(dtype) for n, s in
           [("ff.gate_proj.weight", (inter, hid)), ("ff.up_proj.weight", (inter, hid)), ("ff.down_proj.weight", (hid, inter))]}
    ff.load(DictStore(wts))
    x = torch.randn(rows, hid, generator=g).to(dtype)
    got = ff.forward(x.cuda(), None)
    want = P.swiglu(x.float(), {k: v.float() for k, v in wts.items()}, "ff")
    assert float((got.float().cpu() - want).abs().max()) / float(want.abs().max()) < (1e-5 if dtype == torch.float32 else 2e-2)
    # rotary table: 32-bit angles, (cos, sin) pairs
    rope = POSITION_ENCODINGS.get("rope_neox")(PartSpec("rope_neox", theta=777.0, rotary_dim=12, max_positions=50),
                                               hidden_size=hid, prefix="", dtype=dtype)
    rope.load(DictStore({}))
    cos, sin = P.rope_cos_sin(777.0, 12, torch.arange(50))
    table = rope.table().cpu()
    assert table.shape == (50, 6, 2) and torch.equal(table[..., 0], cos) and torch.equal(table[..., 1], sin)
    assert POSITION_ENCODINGS.get("none")(PartSpec("none"), hidden_size=hid, prefix="", dtype=dtype).table() is None

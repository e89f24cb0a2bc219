"""Toy parts defined here are registered, built into a model beside the attention mixer, and
stepped, without a change to the package: a mixer with fixed-size state of its own (once
deciding on the host per step, once reading only the step's device tensors), a mixer whose
pages hold one vector per token behind a window (not keys and values), a feed-forward that
routes every row to two of five small experts, and a position encoding that is no rotation.  The model's order runs a layer twice (each run with its own
cache and state) and lets one run read the keys and values another run wrote; its ends use
the embedding scale, the head bias and the logit transform, and its attention and
feed-forward carry biases.  Toy parts use torch operations; they exist to test the
framework's seams, not to be a model of anything."""

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DEV = "cuda"
H, NH, NKV, HD, INTER, VOCAB, EPS = 64, 4, 2, 16, 96, 97, 1e-5
WINDOW = 5
EXPERTS, TOP, EXPERT_INTER = 5, 2, 24
EMBED_SCALE, LOGIT_SCALE, LOGIT_CAP = 1.7, 0.5, 3.0


def register_toys():
    from allpaca_b200.parts import CacheNeed, FeedForward, Mixer, PositionEncoding, WeightSpec, register

    class RunningMeanBase(Mixer):
        """y_t = W mean(h_0 .. h_t): needs the sum and the count of a request's earlier rows."""

        def __init__(self, params, env):
            super().__init__(params, env)
            self.hidden = int(params["hidden_size"])
            self.w = None

        def weights(self):
            return {"mean_proj.weight": WeightSpec((self.hidden, self.hidden))}

        def load(self, tensors):
            self.w = tensors["mean_proj.weight"].float()

        def state_bytes(self):
            return (self.hidden + 1) * 4

    @register("mixer", "toy_running_mean_host")
    class RunningMeanHost(RunningMeanBase):
        """Walks the sequences on the host: says so, and is never recorded in a graph."""

        host_control = True

        def forward(self, h, step, cache):
            out = torch.empty(1, step.num_tokens, self.hidden, dtype=torch.float32, device=h.device)
            for s in range(step.num_seqs):
                a, b = step.host_seq_start[s], step.host_seq_start[s + 1]
                state = cache.state[step.host_state_slots[s]].view(torch.float32)
                if step.host_first_position[s] == 0:
                    state.zero_()                                   # a new (or recomputed) request
                x = h[a:b].float()
                sums = state[:self.hidden] + torch.cumsum(x, 0)
                counts = state[self.hidden] + torch.arange(1, b - a + 1, device=h.device)
                out[0, a:b] = (sums / counts[:, None]) @ self.w.T
                state[:self.hidden] = sums[-1]
                state[self.hidden] = counts[-1]
            return out

    @register("mixer", "toy_running_mean_device")
    class RunningMeanDevice(RunningMeanBase):
        """The same from the step's device tensors alone: state rows by ``state_slots``, a
        sequence's first portion known by the position 0 of its first row.  Safe to replay."""

        def forward(self, h, step, cache):
            T, S, Hh = step.num_tokens, step.num_seqs, self.hidden
            ts = step.token_seq.long()
            start = step.seq_start.long()
            slots = step.state_slots.long().clamp(0, cache.state.shape[0] - 1)
            first = step.positions[start[:S].clamp(0, T - 1)] == 0
            rows = cache.state.view(torch.float32)                  # [max_seqs, H + 1]
            held = torch.where(first[:, None], torch.zeros((), device=h.device), rows[slots])
            x = h.float()
            total = torch.cumsum(x, 0)
            before = (total - x)[start[ts]]                         # what precedes the row's own sequence
            sums = held[ts, :Hh] + (total - before)
            counts = held[ts, Hh] + (torch.arange(T, device=h.device) - start[ts] + 1)
            last = (start[1:S + 1] - 1).clamp(0, T - 1)
            rows[slots] = torch.cat([sums[last], counts[last][:, None]], dim=1)
            return ((sums / counts[:, None]) @ self.w.T)[None].contiguous()

    @register("mixer", "toy_window_mean")
    class WindowMean(Mixer):
        """y_t = W mean of the last ``window`` normed rows: its pages hold one 32-bit vector per
        token (no keys, no values, not the engine's type), and pages the window has passed go
        back to the pool.  Reads only device tensors."""

        def __init__(self, params, env):
            super().__init__(params, env)
            self.hidden = int(params["hidden_size"])
            self.window = int(params["window"])
            self.w = None

        def weights(self):
            return {"win_proj.weight": WeightSpec((self.hidden, self.hidden))}

        def load(self, tensors):
            self.w = tensors["win_proj.weight"].float()

        def cache_need(self):
            return CacheNeed(outer=(), inner=(self.hidden,), dtype=torch.float32, window=self.window)

        def forward(self, h, step, cache):
            pages = cache.pages                                     # [num_pages, page, hidden] float32
            n_pages, P = pages.shape[0], pages.shape[1]
            table = step.block_tables[cache.group]
            ts, pos = step.token_seq.long(), step.positions.long()

            def page_of(p):
                return table[ts.view(-1, *[1] * (p.dim() - 1)).expand_as(p),
                             (p // P).clamp(0, table.shape[1] - 1)].long().clamp(0, n_pages - 1)
            pages[page_of(pos), pos % P] = h.float()
            src = pos[:, None] - torch.arange(self.window, device=h.device)[None, :]
            seen = src >= 0
            src = src.clamp(min=0)
            vectors = pages[page_of(src), src % P]                  # [T, window, hidden]
            mean = (vectors * seen[..., None]).sum(1) / seen.sum(1, keepdim=True)
            return (mean @ self.w.T)[None].contiguous()

    @register("feed_forward", "toy_routed")
    class Routed(FeedForward):
        """Every row goes to the ``top`` experts with the largest router logits (32-bit) and
        their outputs are mixed by the softmax over those logits; an expert is
        ``W_out relu(W_in h)``.  Weights with three dimensions."""

        def __init__(self, params, env):
            super().__init__(params, env)
            self.hidden, self.inter = int(params["hidden_size"]), int(params["expert_size"])
            self.experts, self.top = int(params["experts"]), int(params["top"])

        def weights(self):
            return {"router.weight": WeightSpec((self.experts, self.hidden)),
                    "experts.w_in": WeightSpec((self.experts, self.inter, self.hidden)),
                    "experts.w_out": WeightSpec((self.experts, self.hidden, self.inter))}

        def load(self, tensors):
            self.router = tensors["router.weight"].float()
            self.w_in, self.w_out = tensors["experts.w_in"].float(), tensors["experts.w_out"].float()

        def forward(self, h, step):
            x = h.float()
            logits = x @ self.router.T                              # [T, experts]
            best, chosen = logits.topk(self.top, dim=1)
            share = torch.softmax(best, dim=1)
            out = torch.zeros_like(x)
            for e in range(self.experts):                           # no host decision: every expert, masked
                y = torch.relu(x @ self.w_in[e].T) @ self.w_out[e].T
                out += y * (share * (chosen == e)).sum(1, keepdim=True)
            return out[None].contiguous()

    @register("position", "toy_shift")
    class Shift(PositionEncoding):
        """Not a rotation: adds pos * slope to the first element of every query and key head."""

        def __init__(self, params, env):
            super().__init__(params, env)
            self.slope = float(params["slope"])

        def apply(self, q, k, positions):
            q[:, :, 0] += (positions.float() * self.slope).to(q.dtype)[:, None]
            if k is not None:
                k[:, :, 0] += (positions.float() * self.slope).to(k.dtype)[:, None]


def toy_spec(running_mean: str):
    from allpaca_b200.parts import LayerRun, ModelSpec, PartSpec
    norm = PartSpec("rmsnorm", {"size": H, "eps": EPS})

    def block(mixer, ffn_bias=False, routed=False):
        ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": INTER, "bias": ffn_bias})
        if routed:
            ffn = PartSpec("toy_routed", {"hidden_size": H, "expert_size": EXPERT_INTER, "experts": EXPERTS,
                                          "top": TOP})
        return PartSpec("prenorm", {"hidden_size": H, "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm,
                                    "feed_forward_norm": norm, "mixer_prefix": "mix.", "feed_forward_prefix": "mlp.",
                                    "mixer_norm_prefix": "n1.", "feed_forward_norm_prefix": "n2."})
    toy = block(PartSpec(running_mean, {"hidden_size": H}))
    attn = block(PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD,
                                            "qkv_bias": True, "o_bias": True,
                                            "position": PartSpec("rope", {"head_dim": HD, "theta": 1e4})}),
                 ffn_bias=True)
    shifted = block(PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV,
                                               "head_dim": HD, "position": PartSpec("toy_shift", {"slope": 0.01})}),
                    routed=True)
    windowed = block(PartSpec("toy_window_mean", {"hidden_size": H, "window": WINDOW}))
    # no biases, a rotation, a swiglu feed-forward: the block a bfloat16 engine runs with its norms folded in
    bare = block(PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD,
                                            "position": PartSpec("rope", {"head_dim": HD, "theta": 1e4})}))
    return ModelSpec(
        hidden_size=H, vocab_size=VOCAB, layers=(toy, attn, shifted, windowed, bare),
        layer_prefixes=("toy.", "att.", "shf.", "win.", "bar."),
        # toy, attention, toy again (own state), attention again reading the first run's keys, bare attention,
        # shifted, windowed, bare attention again (own cache)
        order=(LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(1, cache_from=1), LayerRun(4), LayerRun(2),
               LayerRun(3), LayerRun(4)),
        final_norm=norm, embedding_name="emb.weight", final_norm_prefix="fn.", head_name="head.weight",
        max_position_embeddings=256, embedding_scale=EMBED_SCALE, head_bias_name="head.bias",
        logit_scale=LOGIT_SCALE, logit_softcap=LOGIT_CAP)


def plain_toy(w, tokens):
    """The same model, whole sequence, plain torch in float64."""
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    pos = torch.arange(T)
    inv = plain_llama.rope_inverse_frequencies(HD, 1e4, None)
    x = w["emb.weight"][torch.tensor(tokens)] * EMBED_SCALE
    kept = {}

    def ffn(x, p, bias=False):
        h = plain_llama.rmsnorm(x, w[p + "n2.weight"], EPS)
        if not bias:
            return x + plain_llama.swiglu_feed_forward(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                                       w[p + "mlp.down_proj.weight"])
        g = h @ w[p + "mlp.gate_proj.weight"].T + w[p + "mlp.gate_proj.bias"]
        u = h @ w[p + "mlp.up_proj.weight"].T + w[p + "mlp.up_proj.bias"]
        return x + (plain_llama.silu(g) * u) @ w[p + "mlp.down_proj.weight"].T + w[p + "mlp.down_proj.bias"]

    def routed(x, p):
        h = plain_llama.rmsnorm(x, w[p + "n2.weight"], EPS)
        logits = h @ w[p + "mlp.router.weight"].T
        out = torch.zeros_like(x)
        for t in range(T):
            best = sorted(range(EXPERTS), key=lambda e: -float(logits[t, e]))[:TOP]
            share = torch.softmax(logits[t, best], 0)
            for s_, e in zip(share, best):
                out[t] += s_ * (torch.relu(h[t] @ w[p + "mlp.experts.w_in"][e].T) @ w[p + "mlp.experts.w_out"][e].T)
        return x + out

    def toy(x):
        h = plain_llama.rmsnorm(x, w["toy.n1.weight"], EPS)
        mean = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
        return ffn(x + mean @ w["toy.mix.mean_proj.weight"].T, "toy.")

    def window_mean(x):
        h = plain_llama.rmsnorm(x, w["win.n1.weight"], EPS)
        mean = torch.stack([h[max(0, t - WINDOW + 1):t + 1].mean(0) for t in range(T)])
        return ffn(x + mean @ w["win.mix.win_proj.weight"].T, "win.")

    def attention(x, p, run, kv_from=None, shift=None, bias=False):
        h = plain_llama.rmsnorm(x, w[p + "n1.weight"], EPS)
        proj = {n: h @ w[p + f"mix.{n}_proj.weight"].T + (w[p + f"mix.{n}_proj.bias"] if bias else 0.0)
                for n in "qkv"}
        q, k, v = proj["q"].view(T, NH, HD), proj["k"].view(T, NKV, HD), proj["v"].view(T, NKV, HD)
        if shift is None:
            q, k = plain_llama.rope_half_split(q, pos, inv), plain_llama.rope_half_split(k, pos, inv)
        else:
            q, k = q.clone(), k.clone()
            q[:, :, 0] += pos.double()[:, None] * shift
            k[:, :, 0] += pos.double()[:, None] * shift
        kept[run] = (k, v)
        if kv_from is not None:
            k, v = kept[kv_from]
        o = plain_llama.causal_attention(q, k, v).reshape(T, -1)
        o = o @ w[p + "mix.o_proj.weight"].T + (w[p + "mix.o_proj.bias"] if bias else 0.0)
        return routed(x + o, p) if shift is not None else ffn(x + o, p, bias)

    x = toy(x)
    x = attention(x, "att.", 1, bias=True)
    x = toy(x)
    x = attention(x, "att.", 3, kv_from=1, bias=True)
    x = attention(x, "bar.", 4)
    x = attention(x, "shf.", 5, shift=0.01)
    x = window_mean(x)
    x = attention(x, "bar.", 7)
    z = (plain_llama.rmsnorm(x, w["fn.weight"], EPS) @ w["head.weight"].T + w["head.bias"]) * LOGIT_SCALE
    return LOGIT_CAP * torch.tanh(z / LOGIT_CAP)


@pytest.mark.parametrize("running_mean,graphs,dtype", [
    ("toy_running_mean_host", True, "float32"), ("toy_running_mean_device", True, "float32"),
    ("toy_running_mean_device", False, "float32"),
    # bfloat16: the attention blocks fold their norms and hand their additions over inside the
    # products' epilogues; the toy blocks beside them take the plain way
    ("toy_running_mean_device", True, "bfloat16"), ("toy_running_mean_host", True, "bfloat16")])
def test_toy_model_is_registered_built_and_stepped(running_mean, graphs, dtype):
    register_toys()
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    from allpaca_b200.models import DecoderModel
    from allpaca_b200.parts import BuildEnv, Workspace, registered
    from allpaca_b200.weights import random_weights

    assert running_mean in registered("mixer") and "toy_window_mean" in registered("mixer")
    assert "toy_shift" in registered("position")
    dev = torch.device(DEV)
    tdtype = getattr(torch, dtype)
    assert "toy_routed" in registered("feed_forward")
    env = BuildEnv(tdtype, dev, Workspace(dev), page_size=8, max_seqs=3)
    model = DecoderModel(toy_spec(running_mean), env)
    weights = random_weights(model, seed=5, dtype=tdtype, device=dev, std=0.08, norm_std=0.02)
    cpu_w = {k: v.cpu() for k, v in weights.items()}           # before loading: the engine may fold norms in
    model.load_weights(weights)
    # cache plan: runs 1, 4, 5 and 7 write keys and values (3 reads 1's), run 6 keeps vectors behind a
    # window in a pool of its own; two runs keep state
    plan = model.cache_plan()
    assert [g.runs for g in plan] == [[1, 4, 5, 7], [6]]
    assert plan[1].need.window == WINDOW and plan[1].need.page_shape(8) == (8, H)
    assert model.state_bytes() == [(H + 1) * 4, 0, (H + 1) * 4, 0, 0, 0, 0, 0]
    assert model.host_control() == (running_mean == "toy_running_mean_host")
    if tdtype == torch.bfloat16:
        # of the attention blocks only the bare one runs folded: biases and the routed toy rule the others out
        assert [b.fused for b in model.blocks] == [False, False, False, False, True]
    runner = ModelRunner(None, EngineConfig(dtype=dtype, page_size=8, num_pages=24, max_num_seqs=3,
                                            max_num_batched_tokens=64, use_cuda_graphs=graphs), model=model)
    assert runner.storages[1].pages.dtype == torch.float32 and runner.storages[1].pages.shape[2:] == (8, H)
    g = torch.Generator().manual_seed(3)
    lengths = (("a", 54), ("b", 30), ("c", 21), ("d", 9), ("e", 12))
    seqs = {r: torch.randint(0, VOCAB, (n,), generator=g).tolist() for r, n in lengths}
    plain = {r: plain_toy(cpu_w, t) for r, t in seqs.items()}

    def check(got, want, what):
        err = float((got.double().cpu() - want).abs().max() / want.abs().max())
        assert err < (1e-4 if tdtype == torch.float32 else 3e-2), (what, err)

    # whole, each alone
    for r, t in seqs.items():
        logits = runner.step([BatchEntry(("whole", r), t, list(range(len(t))))])
        check(logits, plain[r], ("whole", r))
        runner.finish(("whole", r))
    # Portions of some beside single rows of others; "c" starts late in a reused state slot.
    # Then "a" and "b" one row at a time (steps a graph is recorded for, where the parts allow);
    # "b" ends, and "d", whose first step brings one token only, takes over its state slot and its
    # place in the batch: the replayed step must use d's slot, and start d's state from zero.
    done = {r: 0 for r in seqs}
    plan_steps = [[("a", 7)], [("a", 2), ("b", 11)], [("a", 1), ("b", 1)], [("a", 20), ("b", 2)],
                  [("a", 5), ("b", 6)], [("c", 5)], [("c", 16)]]
    plan_steps += [[("a", 1), ("b", 1)]] * 10
    plan_steps += [[("a", 1), ("d", 1)]] * 9
    plan_steps += [[("e", 1)]] * 12
    ended = {"c": 6, "b": 16, "d": 25, "a": 25, "e": 37}       # after which step a request is given back
    for k, rows in enumerate(plan_steps):
        entries = [BatchEntry(("mix", r), seqs[r][done[r]:done[r] + n], list(range(n))) for r, n in rows]
        logits = runner.step(entries)
        at = 0
        for r, n in rows:
            check(logits[at:at + n], plain[r][done[r]:done[r] + n], ("mixed", k, r, done[r]))
            at += n
            done[r] += n
        for r, last in ended.items():
            if last == k:
                runner.finish(("mix", r))
    assert done == {r: n for r, n in lengths}
    runner.cache.check()
    assert runner.cache.num_running() == 0
    if graphs and running_mean == "toy_running_mean_device":
        assert runner.graph_replays >= 10, "decode steps of a model without host control are replayed as graphs"
    else:
        assert runner.graph_replays == 0

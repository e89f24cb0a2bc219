"""A toy mixer with state of its own and a toy position encoding, defined here, are
registered, built into a model beside the attention mixer, and stepped, without a change to
the package.  The model's order runs a layer twice (each run with its own cache and state)
and lets one run read the keys and values another run wrote.  Toy parts use torch
operations; they exist to test the framework's seams, not to be a model of anything."""

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DEV = "cuda"
H, NH, NKV, HD, INTER, VOCAB, EPS = 64, 4, 2, 16, 96, 97, 1e-5


def register_toys():
    from allpaca_b200.parts import Mixer, PositionEncoding, WeightSpec, register

    @register("mixer", "toy_running_mean")
    class RunningMean(Mixer):
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


def toy_spec():
    from allpaca_b200.parts import LayerRun, ModelSpec, PartSpec
    norm = PartSpec("rmsnorm", {"size": H, "eps": EPS})
    ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": INTER})

    def block(mixer):
        return PartSpec("prenorm", {"hidden_size": H, "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm,
                                    "feed_forward_norm": norm, "mixer_prefix": "mix.", "feed_forward_prefix": "mlp.",
                                    "mixer_norm_prefix": "n1.", "feed_forward_norm_prefix": "n2."})
    toy = block(PartSpec("toy_running_mean", {"hidden_size": H}))
    attn = block(PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD,
                                            "position": PartSpec("rope", {"head_dim": HD, "theta": 1e4})}))
    shifted = block(PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV,
                                               "head_dim": HD, "position": PartSpec("toy_shift", {"slope": 0.01})}))
    return ModelSpec(
        hidden_size=H, vocab_size=VOCAB, layers=(toy, attn, shifted),
        layer_prefixes=("toy.", "att.", "shf."),
        # toy, attention, toy again (own state), attention again reading the first run's keys, shifted
        order=(LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(1, cache_from=1), LayerRun(2)),
        final_norm=norm, embedding_name="emb.weight", final_norm_prefix="fn.", head_name="head.weight",
        max_position_embeddings=256)


def plain_toy(w, tokens):
    """The same model, whole sequence, plain torch in float64."""
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    pos = torch.arange(T)
    s = dict(heads=NH, kv_heads=NKV, head_dim=HD)
    inv = plain_llama.rope_inverse_frequencies(HD, 1e4, None)
    x = w["emb.weight"][torch.tensor(tokens)]
    kept = {}

    def ffn(x, p):
        h = plain_llama.rmsnorm(x, w[p + "n2.weight"], EPS)
        return x + plain_llama.swiglu_feed_forward(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                                   w[p + "mlp.down_proj.weight"])

    def toy(x):
        h = plain_llama.rmsnorm(x, w["toy.n1.weight"], EPS)
        mean = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
        return ffn(x + mean @ w["toy.mix.mean_proj.weight"].T, "toy.")

    def attention(x, p, run, kv_from=None, shift=None):
        h = plain_llama.rmsnorm(x, w[p + "n1.weight"], EPS)
        q = (h @ w[p + "mix.q_proj.weight"].T).view(T, NH, HD)
        k = (h @ w[p + "mix.k_proj.weight"].T).view(T, NKV, HD)
        v = (h @ w[p + "mix.v_proj.weight"].T).view(T, NKV, HD)
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
        return ffn(x + o @ w[p + "mix.o_proj.weight"].T, p)

    x = toy(x)
    x = attention(x, "att.", 1)
    x = toy(x)
    x = attention(x, "att.", 3, kv_from=1)
    x = attention(x, "shf.", 4, shift=0.01)
    return plain_llama.rmsnorm(x, w["fn.weight"], EPS) @ w["head.weight"].T


def test_toy_model_is_registered_built_and_stepped():
    register_toys()
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    from allpaca_b200.models import DecoderModel
    from allpaca_b200.parts import BuildEnv, Workspace, registered
    from allpaca_b200.weights import random_weights

    assert "toy_running_mean" in registered("mixer") and "toy_shift" in registered("position")
    dev = torch.device(DEV)
    env = BuildEnv(torch.float32, dev, Workspace(dev), page_size=8, max_seqs=3)
    model = DecoderModel(toy_spec(), env)
    weights = random_weights(model, seed=5, dtype=torch.float32, device=dev, std=0.08, norm_std=0.02)
    model.load_weights(weights)
    # cache plan: three runs write keys (1, 3 reads 1's, 4), two runs keep state
    plan = model.cache_plan()
    assert len(plan) == 1 and plan[0].runs == [1, 4]
    assert model.state_bytes() == [(H + 1) * 4, 0, (H + 1) * 4, 0, 0]
    runner = ModelRunner(None, EngineConfig(dtype="float32", page_size=8, num_pages=24, max_num_seqs=3,
                                            max_num_batched_tokens=64, use_cuda_graphs=False), model=model)
    g = torch.Generator().manual_seed(3)
    seqs = {r: torch.randint(0, VOCAB, (n,), generator=g).tolist() for r, n in (("a", 45), ("b", 30), ("c", 21))}
    cpu_w = {k: v.cpu() for k, v in weights.items()}
    plain = {r: plain_toy(cpu_w, t) for r, t in seqs.items()}

    def check(got, want, what):
        err = float((got.double().cpu() - want).abs().max() / want.abs().max())
        assert err < 1e-4, (what, err)

    # whole, each alone
    for r, t in seqs.items():
        logits = runner.step([BatchEntry(("whole", r), t, list(range(len(t))))])
        check(logits, plain[r], ("whole", r))
        runner.finish(("whole", r))
    # portions of some beside single rows of others; "c" starts late in a reused state slot
    done = {r: 0 for r in seqs}
    plan_steps = [[("a", 7)], [("a", 2), ("b", 11)], [("a", 1), ("b", 1)], [("a", 20), ("b", 2)],
                  [("a", 15), ("b", 16)], [("c", 5)], [("c", 16)]]
    for rows in plan_steps:
        entries = [BatchEntry(("mix", r), seqs[r][done[r]:done[r] + n], list(range(n))) for r, n in rows]
        logits = runner.step(entries)
        at = 0
        for r, n in rows:
            check(logits[at:at + n], plain[r][done[r]:done[r] + n], ("mixed", r, done[r]))
            at += n
            done[r] += n
            if done[r] == len(seqs[r]):
                runner.finish(("mix", r))
    assert done == {r: len(t) for r, t in seqs.items()}
    runner.cache.check()
    assert runner.cache.num_running() == 0

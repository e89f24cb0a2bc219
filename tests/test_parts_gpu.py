"""Each part of a layer alone (norm, rotary embedding, linear, attention mixer, feed-forward,
block) against the plain function of the same part, at sizes of its own, in 32-bit and in
bfloat16, with the rows cut into portions so that the mixer reads what earlier steps cached."""

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DEV = "cuda"
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def rel_err(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def env_for(dtype, page_size=8):
    from allpaca_b200.parts import BuildEnv, Workspace
    dev = torch.device(DEV)
    return BuildEnv(dtype=dtype, device=dev, workspace=Workspace(dev), page_size=page_size, max_seqs=4)


class Harness:
    """A cache of one group and hand-made step batches for parts that need them."""

    def __init__(self, env, need, num_pages=64):
        from allpaca_b200.cache import CacheManager, GroupLayout, GroupStorage
        from allpaca_b200.parts import LayerCache
        self.env = env
        self.manager = CacheManager([GroupLayout(env.page_size, num_pages, need.window)], max_seqs=4)
        self.storage = GroupStorage(1, num_pages, need.page_shape(env.page_size), need.dtype or env.dtype,
                                    env.device)
        self.cache = LayerCache(pages=self.storage.run_view(0), group=0, writes=True)

    def step(self, rows):
        """rows: list of (request, number of new rows)."""
        from allpaca_b200.engine.batch import StepBatch
        firsts = []
        for req, n in rows:
            if not self.manager.has(req):
                self.manager.begin(req)
            firsts.append(self.manager.append(req, n))
        width = max(len(self.manager.block_table(r, 0)) for r, _ in rows)
        table = torch.full((len(rows), width), -1, dtype=torch.int32)
        positions, token_seq, starts = [], [], [0]
        for s, (req, n) in enumerate(rows):
            t = self.manager.block_table(req, 0)
            table[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
            positions += list(range(firsts[s], firsts[s] + n))
            token_seq += [s] * n
            starts.append(starts[-1] + n)
        T = len(positions)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)   # noqa: E731
        batch = StepBatch(
            num_tokens=T, num_seqs=len(rows), num_logit_rows=0, token_ids=i32([0] * T),
            positions=i32(positions), token_seq=i32(token_seq), seq_start=i32(starts),
            context_lens=i32([f + n for f, (_, n) in zip(firsts, rows)]),
            state_slots=i32([self.manager.state_slot(r) for r, _ in rows]), logit_rows=i32([]),
            block_tables=[table.to(DEV)], host_seq_start=starts, host_first_position=firsts,
            host_query_lens=[n for _, n in rows],
            host_state_slots=[self.manager.state_slot(r) for r, _ in rows],
            max_query_len=max(n for _, n in rows), max_context_len=max(f + n for f, (_, n) in zip(firsts, rows)))
        return batch

    def after(self, rows):
        for req, _ in rows:
            self.manager.release_passed(req)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from allpaca_b200.parts import PartSpec, build
    env = env_for(dtype)
    norm = build("norm", PartSpec("rmsnorm", {"size": 200, "eps": 3e-6}), env)
    assert norm.weights()["weight"].shape == (200,)
    w = (1 + 0.1 * torch.randn(200)).to(dtype)
    norm.load({"weight": w.to(DEV)})
    x = torch.randn(6, 200) * 2
    delta = torch.randn(2, 6, 200)
    xd, out = x.to(DEV).clone(), torch.empty(6, 200, dtype=dtype, device=DEV)
    norm.forward(xd, out, delta=delta.to(DEV))
    v = x.double() + delta.double().sum(0)
    assert rel_err(xd, v) < 1e-6
    assert rel_err(out, plain_llama.rmsnorm(v, w.double(), 3e-6)) < (1e-5 if dtype == torch.float32 else 5e-3)


def test_rotary_part_tables_and_sharing():
    from allpaca_b200.engine.batch import StepBatch
    from allpaca_b200.parts import PartSpec, build
    env = env_for(torch.float32)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    a = build("position", PartSpec("rope", {"head_dim": 48, "theta": 500000.0, "scaling": scaling}), env)
    b = build("position", PartSpec("rope", {"head_dim": 48, "theta": 500000.0, "scaling": scaling}), env)
    c = build("position", PartSpec("rope", {"head_dim": 48, "theta": 10000.0, "scaling": None}), env)
    ref = plain_llama.rope_inverse_frequencies(48, 500000.0, scaling)
    assert torch.allclose(a.inv_freq.cpu().double(), ref, rtol=1e-6)
    positions = torch.tensor([0, 1, 77, 300], dtype=torch.int32, device=DEV)
    step = StepBatch(4, 1, 0, positions, positions, positions, positions, positions, positions, positions, [])
    ta, pa = a.rotation_for(step)
    tb, _ = b.rotation_for(step)
    tc, _ = c.rotation_for(step)
    assert ta.data_ptr() == tb.data_ptr() and ta.data_ptr() != tc.data_ptr() and pa == 0
    ang = positions.cpu().float()[:, None] * a.inv_freq.cpu()[None, :]
    assert torch.allclose(ta[..., 0].cpu(), torch.cos(ang.double()).float(), atol=2e-6)
    assert torch.allclose(ta[..., 1].cpu(), torch.sin(ang.double()).float(), atol=2e-6)
    with pytest.raises(ValueError):
        build("position", PartSpec("rope", {"head_dim": 48, "theta": 1e4, "pairing": "spiral"}), env)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("K,N", [(120, 200), (72, 301), (68, 96)])
def test_linear_part_every_consumer_kind(dtype, K, N):
    from allpaca_b200.parts.linear import Linear
    env = env_for(dtype)
    lin = Linear(env, N, K)
    w = (torch.randn(N, K) * 0.1).to(dtype)
    lin.load(w.to(DEV))
    for T in (3, 40, 200):
        a = torch.randn(T, K).to(dtype)
        ref = a.double() @ w.double().T
        delta = lin.forward(a.to(DEV), "t.delta", "delta")
        assert delta.dim() == 3 and delta.dtype == torch.float32
        assert rel_err(delta.sum(0), ref) < 1e-5
        either = lin.forward(a.to(DEV), "t.either", "either")
        got = either.sum(0) if either.dim() == 3 else either
        assert rel_err(got, ref) < (1e-5 if either.dtype == torch.float32 else 5e-3)
        logits = lin.forward(a.to(DEV), "t.logits", "float32")
        assert logits.dtype == torch.float32 and tuple(logits.shape) == (T, N)
        assert rel_err(logits, ref) < 1e-5
    # K = 68 is no multiple of 8: bfloat16 must fall back to the CUDA-core kernel, silently right
    assert lin.uses_tensor_cores() == (dtype == torch.bfloat16 and K % 8 == 0)


def mixer_weights(hidden, nh, nkv, hd, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    shapes = {"q_proj.weight": (nh * hd, hidden), "k_proj.weight": (nkv * hd, hidden),
              "v_proj.weight": (nkv * hd, hidden), "o_proj.weight": (hidden, nh * hd)}
    return {n: (torch.randn(s, generator=g) * 0.08).to(dtype) for n, s in shapes.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,nh,nkv,hd,window", [(96, 3, 1, 32, None), (120, 6, 3, 48, None),
                                                     (64, 4, 2, 16, 24), (200, 5, 5, 80, None)])
def test_attention_mixer_in_portions(dtype, hidden, nh, nkv, hd, window):
    from allpaca_b200.parts import PartSpec, build
    env = env_for(dtype)
    rope = PartSpec("rope", {"head_dim": hd, "theta": 25000.0, "scaling": None})
    mixer = build("mixer", PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "position": rope,
        "window": window}), env)
    w = mixer_weights(hidden, nh, nkv, hd, dtype, seed=hd)
    assert {n: s.shape for n, s in mixer.weights().items()} == {n: tuple(t.shape) for n, t in w.items()}
    mixer.load({n: t.to(DEV) for n, t in w.items()})
    need = mixer.cache_need()
    assert (need.outer, need.inner, need.window) == ((2, nkv), (hd,), window)
    h = Harness(env, need)
    g = torch.Generator().manual_seed(1)
    seqs = {"a": torch.randn(70, hidden, generator=g).to(dtype), "b": torch.randn(33, hidden, generator=g).to(dtype)}
    # portions: a whole prompt chunk beside decode rows of the other, cut at odd places
    plan = [[("a", 17)], [("a", 2), ("b", 30)], [("a", 1), ("b", 1)], [("a", 50), ("b", 2)]]
    done = {k: 0 for k in seqs}
    outs = {k: [] for k in seqs}
    for rows in plan:
        step = h.step(rows)
        x = torch.cat([seqs[r][done[r]:done[r] + n] for r, n in rows]).to(DEV)
        delta = mixer.forward(x, step, h.cache)
        y = delta.sum(0).cpu()
        at = 0
        for r, n in rows:
            outs[r].append(y[at:at + n])
            at += n
            done[r] += n
        h.after(rows)
    s = dict(heads=nh, kv_heads=nkv, head_dim=hd)
    inv = plain_llama.rope_inverse_frequencies(hd, 25000.0, None)
    rt = torch.bfloat16 if dtype == torch.bfloat16 else None
    for r, x in seqs.items():
        wf = {"p." + n: t.float() for n, t in w.items()}
        ref = plain_llama.attention_mixer(x.float(), torch.arange(x.shape[0]), wf, "p.", s, inv.float(), rt,
                                          window=window)
        assert rel_err(torch.cat(outs[r]), ref) < TOL[dtype], r


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from allpaca_b200.parts import PartSpec, build
    env = env_for(dtype)
    ffn = build("feed_forward", PartSpec("swiglu", {"hidden_size": 120, "intermediate_size": 200}), env)
    g = torch.Generator().manual_seed(4)
    w = {"gate_proj.weight": torch.randn(200, 120, generator=g) * 0.1,
         "up_proj.weight": torch.randn(200, 120, generator=g) * 0.1,
         "down_proj.weight": torch.randn(120, 200, generator=g) * 0.1}
    w = {n: t.to(dtype) for n, t in w.items()}
    ffn.load({n: t.to(DEV) for n, t in w.items()})
    for T in (1, 9, 130):
        x = torch.randn(T, 120, generator=g).to(dtype)
        got = ffn.forward(x.to(DEV), None).sum(0)
        ref = plain_llama.swiglu_feed_forward(x.float(), w["gate_proj.weight"].float(), w["up_proj.weight"].float(),
                                              w["down_proj.weight"].float(),
                                              torch.bfloat16 if dtype == torch.bfloat16 else None)
        assert rel_err(got, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prenorm_block(dtype):
    from allpaca_b200.parts import PartSpec, build
    hidden, nh, nkv, hd, inter, eps = 96, 3, 1, 32, 136, 1e-6
    env = env_for(dtype)
    norm = PartSpec("rmsnorm", {"size": hidden, "eps": eps})
    block = build("block", PartSpec("prenorm", {
        "hidden_size": hidden,
        "mixer": PartSpec("gqa_attention", {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv,
                                            "head_dim": hd,
                                            "position": PartSpec("rope", {"head_dim": hd, "theta": 1e4})}),
        "feed_forward": PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}),
        "mixer_norm": norm, "feed_forward_norm": norm, "mixer_prefix": "self_attn.", "feed_forward_prefix": "mlp.",
        "mixer_norm_prefix": "input_layernorm.", "feed_forward_norm_prefix": "post_attention_layernorm."}), env)
    g = torch.Generator().manual_seed(9)
    w = {}
    for prefix, part in block.sub_parts().items():
        for name, ws in part.weights().items():
            t = torch.randn(ws.shape, generator=g) * 0.08
            if ws.role == "norm":
                t = 1 + t
            w[prefix + name] = t.to(dtype)
        part.load({name: w[prefix + name].to(DEV) for name in part.weights()})
    block.finalize()            # bfloat16: the norms' weights go into the products that follow them
    h = Harness(env, block.mixer.cache_need())
    x0 = torch.randn(41, hidden, generator=g)
    x = x0.to(DEV).clone()
    pending = torch.randn(1, 41, hidden, generator=g)            # what an earlier block left to be added
    outs, at = [], 0
    for n in (20, 1, 18, 2):
        step = h.step([("s", n)])
        xs = x[at:at + n].clone()
        d = block.forward(xs, pending[:, at:at + n].to(DEV).contiguous(), step, h.cache)
        # what comes back is a 32-bit delta still to be added, or nothing of the kind where the
        # block's last product has added into the residual itself (None, or the Deferred hand-over
        # of steps of few rows)
        outs.append((xs + d.sum(0) if isinstance(d, torch.Tensor) else xs).cpu())
        at += n
    # the plain block
    wf = {"p." + n: t.float() for n, t in w.items()}
    s = dict(heads=nh, kv_heads=nkv, head_dim=hd)
    inv = plain_llama.rope_inverse_frequencies(hd, 1e4, None).float()
    rt = torch.bfloat16 if dtype == torch.bfloat16 else None
    xr = x0 + pending[0]
    hn = plain_llama._round(plain_llama.rmsnorm(xr, wf["p.input_layernorm.weight"], eps), rt)
    xr = xr + plain_llama.attention_mixer(hn, torch.arange(41), wf, "p.self_attn.", s, inv, rt)
    hn = plain_llama._round(plain_llama.rmsnorm(xr, wf["p.post_attention_layernorm.weight"], eps), rt)
    xr = xr + plain_llama.swiglu_feed_forward(hn, wf["p.mlp.gate_proj.weight"], wf["p.mlp.up_proj.weight"],
                                              wf["p.mlp.down_proj.weight"], rt)
    assert rel_err(torch.cat(outs), xr) < TOL[dtype]


def test_unknown_part_names_are_reported():
    from allpaca_b200.parts import PartError, PartSpec, build
    env = env_for(torch.float32)
    with pytest.raises(PartError, match="gqa_attention"):
        build("mixer", PartSpec("mamba", {}), env)
    with pytest.raises(PartError, match="lacks parameters"):
        build("norm", PartSpec("rmsnorm", {"size": 8}), env)

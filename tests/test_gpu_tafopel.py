"""Tafopel on the GPU against the plain implementation (oracle/tafopel_ref.py, float64, whole sequences, no cache):
every mechanism alone, then whole models through the engine's runner, scheduler bookkeeping and cache / state manager --
prompts, token-by-token decoding, portions, mixed batches, reused pages and slots -- and greedy generation through LLM."""
import math

import pytest
import torch

import tafopel_helpers as th
from oracle import tafopel_ref as ref

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-4, "bfloat16": 6e-2}


def rel_err(got, want):
    """RMS of the difference over the RMS of the expected values."""
    got, want = got.double().cpu(), want.double().cpu()
    return (torch.sqrt(((got - want) ** 2).mean()) / torch.sqrt((want ** 2).mean()).clamp_min(1e-30)).item()


def dev(W, dtype):
    return {k: v.to("cuda", dtype) for k, v in W.items()}


def spans_varlen(q_lens, k_lens):
    from nanovllm import mixops
    cu = lambda v: torch.tensor([0] + list(torch.tensor(v).cumsum(0)), dtype=torch.int32, device="cuda")
    return mixops.StepSpans(len(q_lens), max(q_lens), cu(q_lens), cu(k_lens), None)


# ---------------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cols", [48, 200, 1000])
def test_residual_update_and_layer_norm(dtype, cols):
    from nanovllm import mixops
    g = torch.Generator().manual_seed(cols)
    x = torch.randn(7, cols, generator=g) * 3 + 1.5
    a = torch.randn(7, cols, generator=g).to(DT[dtype])
    b = torch.randn(7, cols, generator=g).to(DT[dtype])
    b32 = torch.randn(7, cols, generator=g)
    w = (1 + 0.3 * torch.randn(cols, generator=g)).to(DT[dtype])
    xd = x.cuda()
    out = mixops.add_layernorm(xd, w.cuda(), 1e-5, a=a.cuda(), b=b.cuda(), b32=b32.cuda())
    want_x = x.double() + (a.double() + b.double() + b32.double())
    assert rel_err(xd, want_x) < 1e-6                                   # the stream itself stays fp32 in both formats
    assert rel_err(out, ref.layer_norm(want_x, w.double(), 1e-5)) < (2e-6 if dtype == "float32" else 4e-3)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    sel = mixops.add_layernorm(xd, w.cuda(), 1e-5, rows_idx=rows)
    assert torch.equal(sel, out[[5, 0, 5]])


def plain_sink_attention(q, rows, rank, sink, scale, pos):
    """q [H, D], rows [L, D] (latent | shared key part): softmax over rows[: pos + 1] and the sink, values = rows[:, :rank]."""
    s = (q.double() @ rows[:pos + 1].double().T) * scale
    top = torch.maximum(s.max(-1, keepdim=True).values, sink.double()[:, None])
    e = torch.exp(s - top)
    p = e / (e.sum(-1, keepdim=True) + torch.exp(sink.double()[:, None] - top))
    return p @ rows[:pos + 1, :rank].double()


def identity_rotation(max_pos, dims):
    return torch.cat([torch.ones(max_pos, dims // 2), torch.zeros(max_pos, dims // 2)], 1).cuda()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("bs", [16, 64])
def test_attention_kernel_finds_one_far_key_and_respects_edges(dtype, bs):
    """One key is made to dominate (its row is a large multiple of the query): the output must be that key's latent when the key
    is visible, and must not move when it is one position too far.  The key sits at page borders, at position 0, and hundreds
    of tokens back; queries are rows of a portion and single decoded tokens, over pages in a scrambled order that also hold a
    stale dominating row just past the sequence's end."""
    from nanovllm import mixops
    H, rank, rd, L = 3, 40, 8, 420
    D = rank + rd
    g = torch.Generator().manual_seed(7)
    pages = torch.randperm(40, generator=g)[: (L + bs - 1) // bs + 1].to(torch.int32)
    sink = torch.tensor([0.3, -2.0, 1.0])
    cs = identity_rotation(L + 8, rd)
    for star in (0, bs - 1, bs, bs + 1, 3 * bs - 1, 207, L - 1):
        q = torch.randn(H, D, generator=g)
        rows = torch.randn(L + 1, D, generator=g) * 0.3
        rows[star] = 6.0 * q[1] / q[1].norm()                # head 1 looks straight at it; other heads see it as an ordinary key
        rows[L] = 50.0 * q[1]                                # stale row behind the end: never visible
        cache = torch.zeros(40 * bs, D, dtype=DT[dtype])
        for j in range(L + 1):
            cache[int(pages[j // bs]) * bs + j % bs] = rows[j].to(DT[dtype])
        rows_t = torch.stack([cache[int(pages[j // bs]) * bs + j % bs] for j in range(L + 1)]).float()
        bt = pages[None, :].cuda().contiguous()
        for pos in sorted({star - 1, star, star + 1, L - 1} & set(range(L))):
            qt = q.to(DT[dtype])
            q_lat = qt[:, None, :rank].contiguous().cuda()                         # [H, 1, rank]
            q_raw = qt[None, :, :].contiguous().cuda()                             # [1, H, D]: the rotated part starts at `rank`
            want = plain_sink_attention(qt.float(), rows_t, rank, sink, 0.5, pos)
            # decoded alone
            sp = mixops.StepSpans(1, 1, None, None, torch.tensor([pos + 1], dtype=torch.int32, device="cuda"))
            got = mixops.latent_attention(q_lat, q_raw, rank, cache.cuda(), bt, bs, sp, sink.cuda(), cs, 0.5)[:, 0]
            assert rel_err(got, want) < (1e-5 if dtype == "float32" else 1e-2), (star, pos, "decode")
            if pos >= star:
                assert rel_err(got[1], rows_t[star, :rank]) < 0.05
            # as the last row of a 5-token portion whose other rows are other queries
            n = min(5, pos + 1)
            ql = torch.randn(H, n, rank, generator=g).to(DT[dtype])
            qr = torch.randn(n, H, D, generator=g).to(DT[dtype])
            ql[:, n - 1], qr[n - 1] = qt[:, :rank], qt
            sp = spans_varlen([n], [pos + 1])
            got = mixops.latent_attention(ql.cuda(), qr.cuda(), rank, cache.cuda(), bt, bs, sp, sink.cuda(), cs, 0.5)
            assert rel_err(got[:, n - 1], want) < (1e-5 if dtype == "float32" else 1e-2), (star, pos, "portion")
            if n > 1:                                        # and the row before it sees one key less
                full = torch.cat([ql[:, n - 2].float(), qr[n - 2, :, rank:].float()], 1)
                assert rel_err(got[:, n - 2], plain_sink_attention(full, rows_t, rank, sink, 0.5, pos - 1)) < (1e-5 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("bs", [16, 64])
@pytest.mark.parametrize("shape", [(6, 192, 16), (20, 64, 32), (8, 512, 64), (16, 256, 64), (1, 24, 2), (12, 80, 16)])
def test_attention_kernel_shapes_and_batches(shape, bs):
    """Head counts on both sides of a warp's 16 rows and of a 64-row tile, latents narrower and wider than one column pass and
    wide enough for the short key tiles; a batch of portions and one of single tokens whose extents end at, just before and
    just after page and key-tile borders.  Every row against the plain softmax, in bf16 (tensor cores, and the FMA form) and fp32."""
    from nanovllm import mixops
    H, rank, rd = shape
    D = rank + rd
    g = torch.Generator().manual_seed(H * 1000 + rank)
    extents = [(5, 70), (64, 64), (1, 129), (130, 260), (2, 2), (33, 192), (3, 65)]          # (tokens in the step, tokens held after it)
    width = max(-(-k // bs) for _, k in extents) + 1
    n_pages = width * len(extents) + 2
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    bt = perm[:width * len(extents)].view(len(extents), width).contiguous()
    sink = torch.randn(H, generator=g)
    cs = identity_rotation(300, rd)
    for dtype, kw, tol in (("bfloat16", {}, 1e-2), ("bfloat16", {"fma": True}, 1e-2), ("float32", {}, 1e-5)):
        cache = (torch.randn(n_pages * bs, D, generator=g) * 0.5).to(DT[dtype])
        rows = [torch.stack([cache[int(bt[s, j // bs]) * bs + j % bs] for j in range(k)]).float() for s, (_, k) in enumerate(extents)]
        # portions
        n = sum(q for q, _ in extents)
        q = (torch.randn(n, H, D, generator=g) * 1.5).to(DT[dtype])
        q_lat = q[:, :, :rank].transpose(0, 1).contiguous()
        sp = spans_varlen([q for q, _ in extents], [k for _, k in extents])
        got = mixops.latent_attention(q_lat.cuda(), q.cuda(), rank, cache.cuda(), bt.cuda(), bs, sp, sink.cuda(), cs, 0.3, **kw)
        at = 0
        for s, (ql, kl) in enumerate(extents):
            for i in range(ql):
                want = plain_sink_attention(q[at + i].float(), rows[s], rank, sink, 0.3, kl - ql + i)
                assert rel_err(got[:, at + i], want) < tol, (dtype, kw, "portion", s, i)
            at += ql
        # single tokens, one padding row (extent 0) in the middle
        lens = [k for _, k in extents]
        lens.insert(3, 0)
        btd = torch.cat([bt[:3], bt[:1], bt[3:]]).contiguous()
        q1 = (torch.randn(len(lens), H, D, generator=g) * 1.5).to(DT[dtype])
        sp = mixops.StepSpans(len(lens), 1, None, None, torch.tensor(lens, dtype=torch.int32, device="cuda"))
        got = mixops.latent_attention(q1[:, :, :rank].transpose(0, 1).contiguous().cuda(), q1.cuda(), rank, cache.cuda(), btd.cuda(), bs, sp,
                                      sink.cuda(), cs, 0.3, **kw)
        for r, kl in enumerate(lens):
            if kl:
                s = r if r < 3 else r - 1
                assert rel_err(got[:, r], plain_sink_attention(q1[r].float(), rows[s], rank, sink, 0.3, kl - 1)) < tol, (dtype, kw, "single", r)


def test_a_large_sink_takes_the_weight():
    from nanovllm import mixops
    H, rank, rd, bs = 2, 12, 4, 16
    g = torch.Generator().manual_seed(1)
    cache = torch.randn(4 * bs, rank + rd, generator=g).cuda()
    q_lat, q_raw = torch.randn(H, 1, rank, generator=g).cuda(), torch.randn(1, H, rank + rd, generator=g).cuda()
    bt = torch.tensor([[2, 0]], dtype=torch.int32, device="cuda")
    sp = mixops.StepSpans(1, 1, None, None, torch.tensor([20], dtype=torch.int32, device="cuda"))
    sink = torch.tensor([30.0, -30.0]).cuda()
    out = mixops.latent_attention(q_lat, q_raw, rank, cache, bt, bs, sp, sink, identity_rotation(32, rd), 0.3)[:, 0]
    assert out[0].abs().max() < 1e-6 and out[1].abs().max() > 1e-2
    rows = torch.cat([cache[2 * bs:3 * bs], cache[:4]]).cpu()
    q = torch.cat([q_lat[:, 0], q_raw[0, :, rank:]], 1).cpu()
    assert rel_err(out, plain_sink_attention(q, rows, rank, sink.cpu(), 0.3, 19)) < 1e-5


def _latent_layer(m, width, dtype, W, pre, max_pos=512):
    from nanovllm.layers.latent_attention import LatentAttention
    la = LatentAttention(width, m, 1e-5, DT[dtype], torch.device("cuda"), max_pos)
    for k, v in W.items():
        if k.startswith(pre):
            assert la.load(k[len(pre):], v.to("cuda", DT[dtype]) if k != pre + "sink" else v.cuda())
    return la


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_attention_layer_in_portions_over_scrambled_pages(dtype):
    from nanovllm.utils.context import reset_context, set_context
    cfg = th.config([(th.latent(), None)])
    W = th.random_weights(cfg, 11)
    m, width, bs, L = cfg["layers"][0]["mixer"], cfg["width"], 16, 75
    la = _latent_layer(m, width, dtype, W, "l0.mix.")
    la.cache = torch.zeros(8 * bs, m["kv_rank"] + m["rot_dim"], dtype=DT[dtype], device="cuda")
    la.block_size = bs
    h = torch.randn(L, width, generator=torch.Generator().manual_seed(5)).to(DT[dtype])
    W64 = {k: v.double() for k, v in W.items()}
    want = ref.latent_attention(h.double(), W64, "l0.mix.", m, 1e-5, ref.latent_kv(h.double(), W64, "l0.mix.", m, 1e-5))
    pages = [6, 1, 4, 0, 3]
    bt = torch.tensor([pages], dtype=torch.int32, device="cuda")
    got, at = [], 0
    for n in (33, 2, 1, 1, 17, 2, 19):                       # portions cut inside pages, down to two tokens and single tokens
        pos = torch.arange(at, at + n, dtype=torch.int64, device="cuda")
        slots = torch.tensor([pages[p // bs] * bs + p % bs for p in range(at, at + n)], dtype=torch.int32, device="cuda")
        sp = spans_varlen([n], [at + n])
        set_context(True, sp.cu_q, sp.cu_k, n, at + n, slots, None, bt)
        from nanovllm.utils.context import get_context
        got.append(la.forward(h[at:at + n].cuda(), pos, get_context(), sp))
        at += n
    reset_context()
    assert rel_err(torch.cat(got), want) < (2e-5 if dtype == "float32" else 3e-2)


def _scan_layer(m, width, dtype, W, pre, slots):
    from nanovllm.layers.selective_scan import SelectiveScanMixer
    mx = SelectiveScanMixer(width, m, DT[dtype], torch.device("cuda"))
    for k, v in W.items():
        if k.startswith(pre):
            assert mx.load(k[len(pre):], v.to("cuda", DT[dtype]))
    mx.bind_state(slots)
    mx.conv_state.fill_(7.0)          # what an earlier owner left behind must not be read by a new sequence
    mx.ssm_state.fill_(-3.0)
    return mx


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(inner=48, state=6, dt_rank=5, conv=4), dict(inner=70, state=33, dt_rank=1, conv=1),
                                   dict(inner=33, state=1, dt_rank=9, conv=6), dict(inner=136, state=128, dt_rank=4, conv=9),
                                   dict(inner=300, state=16, dt_rank=12, conv=3), dict(inner=64, state=72, dt_rank=2, conv=2)])
def test_selective_scan_layer_portions_batches_and_dirty_slots(dtype, shape):
    from types import SimpleNamespace
    cfg = th.config([(th.mamba(**shape), None)])
    W = th.random_weights(cfg, 2)
    m, width = cfg["layers"][0]["mixer"], cfg["width"]
    mx = _scan_layer(m, width, dtype, W, "l0.mix.", 3)
    g = torch.Generator().manual_seed(9)
    ha, hb = torch.randn(41, width, generator=g).to(DT[dtype]), torch.randn(23, width, generator=g).to(DT[dtype])
    W64 = {k: v.double() for k, v in W.items()}
    want_a, want_b = ref.mamba1(ha.double(), W64, "l0.mix.", m), ref.mamba1(hb.double(), W64, "l0.mix.", m)
    tol = 2e-5 if dtype == "float32" else 3e-2

    def run(parts):                                          # parts: [(h rows, tokens behind them, slot)]
        q, k = [p[0].shape[0] for p in parts], [p[0].shape[0] + p[1] for p in parts]
        ctx = SimpleNamespace(state_slots=torch.tensor([p[2] for p in parts], dtype=torch.int32, device="cuda"))
        return mx.forward(torch.cat([p[0] for p in parts]).cuda(), None, ctx, spans_varlen(q, k))

    # a alone in slot 2, in portions that are shorter than the convolution, then long, then single tokens
    outs, at = [], 0
    for n in (1, 2, 3, 1, 20, 1, 1, 12):
        outs.append(run([(ha[at:at + n], at, 2)]))
        at += n
    assert rel_err(torch.cat(outs), want_a) < tol
    # b starts in the same slot right after a (its state must start from zero), beside a second copy of a in slot 0
    o1 = run([(hb[:7], 0, 2), (ha[:30], 0, 0)])
    o2 = run([(ha[30:31], 30, 0), (hb[7:], 7, 2)])           # a decodes one token beside a portion of b
    assert rel_err(torch.cat([o1[:7], o2[1:]]), want_b) < tol
    assert rel_err(torch.cat([o1[7:], o2[:1]]), want_a[:31]) < tol
    # decode form (one token per row, a padding row in the middle)
    from nanovllm import mixops
    ctx = SimpleNamespace(state_slots=torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda"))
    sp = mixops.StepSpans(3, 1, None, None, torch.tensor([32, 0, 0], dtype=torch.int32, device="cuda"))
    o3 = mx.forward(torch.stack([ha[31], ha[0], ha[1]]).cuda(), None, ctx, sp)
    assert rel_err(o3[0], want_a[31]) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mlp", [th.moe(5, 2, 40, 24), th.moe(3, 1, 24, 0), th.moe(9, 4, 70, 8), th.dense(72)])
def test_feed_forward_blocks(dtype, mlp):
    from nanovllm.layers.moe import GatedDenseFF, RoutedExpertsFF
    cfg = th.config([(th.mamba(), mlp)])
    W = th.random_weights(cfg, 4)
    width = cfg["width"]
    ff = (GatedDenseFF if mlp["kind"] == "dense" else RoutedExpertsFF)(width, mlp, DT[dtype], torch.device("cuda"))
    for k, v in W.items():
        if k.startswith("l0.mlp."):
            assert ff.load(k[7:], v.to("cuda", DT[dtype]))
    h = torch.randn(77, width, generator=torch.Generator().manual_seed(3)).to(DT[dtype])
    W64 = {k: v.double() for k, v in W.items()}
    want = ref.dense_ff(h.double(), W64, "l0.mlp.") if mlp["kind"] == "dense" else ref.moe_ff(h.double(), W64, "l0.mlp.", mlp)
    t, f32 = ff.forward(h.cuda())
    assert rel_err(t if t is not None else f32, want) < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("experts,top", [(1, 1), (8, 8), (16, 2), (33, 5), (64, 6), (200, 8)])
def test_router_picks_the_largest_and_survives_bad_logits(experts, top):
    """The chosen experts are those of a plain top-k (equal logits: the lower index), with their sigmoid as weight; rows that hold
    NaN or infinities still get `top` distinct experts in range (such rows occur in warm-up steps over an unwritten cache)."""
    from nanovllm import mixops
    g = torch.Generator().manual_seed(experts)
    z = torch.randn(50, experts + 1, generator=g)                    # one more column than experts: a strided view, as in the layer
    z[7] = 0.25                                                      # all equal
    idx, w = mixops.moe_route(z.cuda()[:, :experts], experts, top)
    want = torch.topk(z[:, :experts], top, dim=1)
    assert torch.equal(idx.cpu().long()[:7], want.indices[:7]) and torch.equal(idx.cpu().long()[8:], want.indices[8:])
    assert idx[7].tolist() == list(range(top))
    assert rel_err(w, torch.sigmoid(want.values)) < 1e-6
    bad = z.clone()
    bad[::3] = float("nan")
    bad[1, ::2] = float("nan")
    bad[2] = float("inf")
    bad[4] = -float("inf")
    idx, _ = mixops.moe_route(bad.cuda()[:, :experts], experts, top)
    idx = idx.cpu()
    assert int(idx.min()) >= 0 and int(idx.max()) < experts
    assert all(len(set(row.tolist())) == top for row in idx)


def test_expert_weight_scales_the_input_not_the_output():
    """relu(w x)^2 = w^2 relu(x)^2: with one expert and no shared expert the output is w^2 times the unweighted expert."""
    from nanovllm.layers.moe import RoutedExpertsFF
    mlp = th.moe(1, 1, 16, 0)
    ff = RoutedExpertsFF(32, mlp, torch.float32, torch.device("cuda"))
    g = torch.Generator().manual_seed(0)
    up, down, router = torch.randn(16, 32, generator=g), torch.randn(32, 16, generator=g), torch.randn(1, 32, generator=g)
    ff.load("e0.up", up.cuda()), ff.load("e0.down", down.cuda()), ff.load("router", router.cuda())
    h = torch.randn(5, 32, generator=g)
    w = torch.sigmoid(h @ router.T)
    want = (w ** 2) * ref.relu2_expert(h, up, down)
    assert rel_err(ff.forward(h.cuda())[1], want) < 1e-5


# ---------------------------------------------------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------------------------------------------------
class Replay:
    """The engine in logits-only mode: dictated steps through Scheduler.plan_step and ModelRunner.run_logits."""

    def __init__(self, path, dtype, pool_tokens=320, block=16, seqs=4, eager=False):
        from nanovllm.config import Config
        from nanovllm.engine.model_runner import ModelRunner
        from nanovllm.engine.scheduler import Scheduler
        from nanovllm.engine.sequence import Sequence
        from nanovllm.models.registry import read_config
        cfg = Config(path, hf_config=read_config(path), max_num_seqs=seqs, max_num_batched_tokens=pool_tokens, max_model_len=pool_tokens,
                     kvcache_block_size=block, num_kvcache_blocks=pool_tokens // block, enforce_eager=eager, dtype=dtype, logits_only=True)
        Sequence.block_size = block
        self.Sequence, self.block = Sequence, block
        self.runner, self.sched, self.live = ModelRunner(cfg, 0, None), Scheduler(cfg), {}

    def step(self, entries):
        """entries: [(id, tokens)] -> {id: logits of all its tokens in this step}"""
        self.Sequence.block_size = self.block
        portions, n = [], 0
        for rid, toks in entries:
            seq = self.live.get(rid)
            if seq is None:
                seq = self.live[rid] = self.Sequence(list(toks))
            portions.append((seq, list(toks)))
            n += len(toks)
        batch, varlen = self.sched.plan_step(portions)
        lg = self.runner.run_logits(batch, varlen, list(range(n)) if varlen else None)
        self.sched.postprocess_replay(batch)
        out, at = {}, 0
        for rid, toks in entries:
            out[rid] = lg[at:at + len(toks)]
            at += len(toks)
        return out

    def end(self, rid):
        self.sched.retire(self.live.pop(rid))


@pytest.fixture(scope="module")
def checkpoints(tmp_path_factory):
    root = tmp_path_factory.mktemp("tafopel")
    out = {}
    for name, cfg in (("a", th.config_a()), ("b", th.config_b()), ("c", th.config_c()), ("d", th.config_d()), ("e", th.config_e())):
        W = th.random_weights(cfg, 21)
        out[name] = (th.write_checkpoint(str(root / name), cfg, W), cfg, W)
    return out


@pytest.fixture(scope="module")
def engines(checkpoints):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = Replay(checkpoints[name][0], dtype)
        return made[(name, dtype)]
    yield get
    for e in made.values():
        e.runner.exit()


def oracle_logits(checkpoints, name, toks):
    _, cfg, W = checkpoints[name]
    return ref.forward(cfg, W, toks)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_whole_prompt_and_first_tokens(engines, checkpoints, name, dtype):
    e = engines(name, dtype)
    vocab = checkpoints[name][1]["vocab"]
    for i, n in enumerate((1, 2, 17, 150)):
        toks = th.tokens(n, vocab, i)
        got = e.step([("p", toks)])["p"]
        e.end("p")
        assert rel_err(got, oracle_logits(checkpoints, name, toks)) < TOL[dtype], n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_long_decoding_matches_the_prompt_path(engines, checkpoints, name, dtype):
    """One prompt token, then 170 tokens one by one through the decode graphs, across ten pages."""
    e = engines(name, dtype)
    toks = th.tokens(171, checkpoints[name][1]["vocab"], 5)
    want = oracle_logits(checkpoints, name, toks)
    got = [e.step([("d", toks[:1])])["d"]]
    for t in toks[1:]:
        got.append(e.step([("d", [t])])["d"])
    e.end("d")
    got = torch.cat(got)
    assert rel_err(got, want) < TOL[dtype]
    assert rel_err(got[-20:], want[-20:]) < TOL[dtype]       # no drift at the far end


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_portions_of_many_sizes(engines, checkpoints, name, dtype):
    e = engines(name, dtype)
    cuts = (2, 3, 2, 31, 16, 2, 1, 1, 48, 15, 1, 5, 33)
    toks = th.tokens(sum(cuts), checkpoints[name][1]["vocab"], 6)
    got, at = [], 0
    for n in cuts:
        got.append(e.step([("c", toks[at:at + n])])["c"])
        at += n
    e.end("c")
    assert rel_err(torch.cat(got), oracle_logits(checkpoints, name, toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(engines, checkpoints, name, dtype):
    """Four requests of unequal length, portions beside single tokens; two of them end early and a fifth and sixth take over
    their pages and state slots while the others go on.  Every request must come out as if it had run alone."""
    e = engines(name, dtype)
    vocab = checkpoints[name][1]["vocab"]
    T = {k: th.tokens(n, vocab, 10 + i) for i, (k, n) in enumerate(dict(a=90, b=37, c=9, d=140, e=70, f=44).items())}
    plan = [
        [("a", 40), ("b", 2)], [("a", 1), ("b", 30), ("c", 9)], [("a", 1), ("b", 1), ("d", 64)], [("a", 1), ("b", 1), ("d", 1)],
        [("a", 17), ("b", 3), ("d", 2)], [("a", 1), ("d", 1)], [("a", 29), ("d", 72)],
        # b and c are done: e and f arrive in their places
        [("e", 33), ("f", 1), ("d", 0)], [("e", 1), ("f", 43)], [("e", 36)],
    ]
    got = {k: [] for k in T}
    at = {k: 0 for k in T}
    ended = set()
    for step in plan:
        entries = [(k, T[k][at[k]:at[k] + n]) for k, n in step if n]
        for k, n in step:
            at[k] += n
        for k, lg in e.step(entries).items():
            got[k].append(lg)
        for k in T:
            if at[k] == len(T[k]) and k in e.live and k not in ended:
                e.end(k)
                ended.add(k)
    assert ended == set(T)
    for k in T:
        assert rel_err(torch.cat(got[k]), oracle_logits(checkpoints, name, T[k])) < TOL[dtype], k


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_of_64_tokens(checkpoints, dtype):
    """Pages as long as the attention kernel's key tile (one page lookup per tile), a prompt in portions and decoding over a page border."""
    e = Replay(checkpoints["a"][0], dtype, pool_tokens=512, block=64, seqs=2)
    toks = th.tokens(200, checkpoints["a"][1]["vocab"], 77)
    got, at = [], 0
    for n in (70, 58, 1, 1, 1, 60, 9):
        got.append(e.step([("p", toks[at:at + n])])["p"])
        at += n
    e.end("p")
    e.runner.exit()
    assert rel_err(torch.cat(got), oracle_logits(checkpoints, "a", toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wider_model_over_64_token_pages(checkpoints, dtype):
    """The larger configuration: a 333-token prompt in portions that end beside page borders, then single tokens, next to a second
    request that arrives in the middle.  In bf16 a rounded router input may swap two nearly equal experts for a token, so the
    bound there is on the median error over positions rather than on the sum."""
    e = Replay(checkpoints["e"][0], dtype, pool_tokens=768, block=64, seqs=3)
    vocab = checkpoints["e"][1]["vocab"]
    a, b = th.tokens(333, vocab, 81), th.tokens(90, vocab, 82)
    got = {"a": [], "b": []}
    at = {"a": 0, "b": 0}
    for step in ([("a", 63)], [("a", 2)], [("a", 64), ("b", 1)], [("a", 1), ("b", 70)], [("a", 130), ("b", 1)], [("a", 1), ("b", 18)], [("a", 60)],
                 *[[("a", 1)] for _ in range(12)]):
        entries = [(k, (a if k == "a" else b)[at[k]:at[k] + n]) for k, n in step]
        for k, n in step:
            at[k] += n
        for k, lg in e.step(entries).items():
            got[k].append(lg)
    e.runner.exit()
    assert at == {"a": 333, "b": 90}
    for k, toks in (("a", a), ("b", b)):
        out, want = torch.cat(got[k]).double().cpu(), oracle_logits(checkpoints, "e", toks)
        if dtype == "float32":
            assert rel_err(out, want) < TOL[dtype], k
        else:
            per_pos = ((out - want) ** 2).mean(1).sqrt() / (want ** 2).mean(1).sqrt()
            assert per_pos.median().item() < 0.04 and rel_err(out, want) < 0.25, k


def test_batch_does_not_change_a_request_beyond_rounding(engines, checkpoints):
    e = engines("a", "float32")
    vocab = checkpoints["a"][1]["vocab"]
    x, y = th.tokens(50, vocab, 30), th.tokens(21, vocab, 31)
    alone = e.step([("x", x)])["x"]
    e.end("x")
    both = e.step([("y", y), ("x", x)])["x"]
    e.end("x"), e.end("y")
    assert rel_err(both, alone) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(checkpoints, dtype):
    """LLM.generate on a checkpoint without a tokenizer: scheduler, block and slot manager, decode graphs, sampler.  Teacher-forced
    against the plain implementation: each generated token is its argmax, or loses to it by less than the format's rounding."""
    from nanovllm import LLM, SamplingParams
    path, cfg, W = checkpoints["a"]
    llm = LLM(path, dtype=dtype, max_num_seqs=3, max_model_len=256, max_num_batched_tokens=96, kvcache_block_size=16,
              num_kvcache_blocks=24, gpu_memory_utilization=0.5)
    prompts = [th.tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate((5, 61, 1, 100, 18))]      # more requests than slots, chunked prompts
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True), use_tqdm=False)
    llm.exit()
    assert [len(o["token_ids"]) for o in outs] == [24] * 5
    tol = 1e-3 if dtype == "float32" else 0.15
    for p, o in zip(prompts, outs):
        seq = p + o["token_ids"]
        lg = ref.forward(cfg, W, seq[:-1])
        for i, tok in enumerate(o["token_ids"]):
            row = lg[len(p) - 1 + i]
            assert (row.max() - row[tok]).item() <= tol * row.std().item(), (len(p), i)


def test_replay_command_line(checkpoints, tmp_path):
    """bin/trace_run end to end: JSON steps on stdin, logits files and 'done' lines out."""
    import json
    import os
    import subprocess
    import numpy as np
    path, cfg, W = checkpoints["b"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = th.tokens(40, cfg["vocab"], 50)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[30:31], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "q", "tokens": toks[31:32], "want": [0]}, {"id": "r", "tokens": toks[:3], "want": [2]}], "end": ["r"]},
             {"step": 3, "entries": [{"id": "q", "tokens": toks[32:], "want": [7]}], "end": ["q"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    want = ref.forward(cfg, W, toks)
    rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
    assert not (out / "1.f32").exists()
    assert rel_err(rd(0), want[[0, 29]]) < 3e-4 and rel_err(rd(3), want[[39]]) < 3e-4
    assert rel_err(rd(2), torch.stack([want[31], want[2]])) < 3e-4

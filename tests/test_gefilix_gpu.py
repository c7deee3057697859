"""The Gefilix design on the GPU against the plain implementation: each mechanism's part alone,
then whole models through the trace replayer in every way of cutting requests into steps, then
greedy generation through the engine and its scheduler."""

import math

import numpy as np
import pytest
import torch

import plain_gefilix as plain
from gefilix_helpers import check, oracle, prompts, write_folder
from helpers import mixed_trace
from test_engine_gpu import step_context
from tiny_gefilix import GEFILIX, calm

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
EPS = 1e-5


def rounded(t):
    return t.bfloat16().float()


def on_device(w, dtype):
    return {k: v.cuda().to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()}


# ---- each mechanism alone -------------------------------------------------------------------


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_after_the_sum_and_the_scaled_embedding(dtype):
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(0)
    d, T, V = 72, 11, 50
    gain = 1 + 0.1 * torch.randn(d, generator=g)
    norm = build_part("norm", PartSpec("stream_rms_norm", dict(eps=EPS, alpha=1.7, tensor="n")), d)
    norm.load({"n": gain.cuda()})
    norm.bind_dtype(dtype)
    x = torch.randn(T, d, generator=g)
    for y, held_as in ((torch.randn(T, d, generator=g), torch.float32), (rounded(torch.randn(T, d, generator=g)), dtype)):
        stream, copy = norm.add_forward(x.cuda(), y.cuda().to(held_as))
        ref = plain.rms_norm(1.7 * x.double() + y.double(), gain.double(), EPS).float()
        check(stream, ref, torch.float32, "the stream after the sum")
        assert stream.dtype == torch.float32 and copy.dtype == dtype
        assert torch.equal(copy.float(), stream.to(dtype).float())
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    last = norm.forward(x.cuda(), rows)
    assert last.dtype == dtype
    check(last, plain.rms_norm(x.double(), gain.double(), EPS).float()[[7, 0, 3]], dtype, "plain norm of chosen rows", 0.01)
    emb = build_part("embedding", PartSpec("scaled_embedding", dict(vocab_size=V, scale=0.3, tensor="e")), d)
    table = rounded(torch.randn(V, d, generator=g))
    emb.load({"e": table.cuda().to(dtype)})
    ids = torch.tensor([4, 49, 0, 4], dtype=torch.int32, device="cuda")
    out = emb.forward(ids)
    assert out.dtype == torch.float32
    check(out, table[[4, 49, 0, 4]] * 0.3, torch.float32, "scaled embedding")


def test_norm_after_the_sum_reading_a_products_partial_sums():
    """With few tokens the last product of a sublayer stays as the GEMM's partial sums and the
    norm's kernel adds them up: the finished product followed by the norm, up to the order in
    which a row's squares are added (a few float32 ulps; the bfloat16 copy within one of its own)."""
    from atomserve_b200 import ops
    from atomserve_b200.ops.linear import PartialSums

    g = torch.Generator().manual_seed(4)
    met = 0
    for T, d, K in ((1, 256, 512), (5, 320, 1024), (8, 2048, 2048), (33, 256, 384)):
        inner = (torch.randn(T, K, generator=g)).bfloat16().cuda()
        w = (torch.randn(d, K, generator=g) * K**-0.5).bfloat16().cuda()
        x = torch.randn(T, d, generator=g).cuda()
        gain = (1 + 0.1 * torch.randn(d, generator=g)).cuda()
        whole = ops.scaled_add_rms_norm(x, ops.linear(inner, w, out_dtype=torch.float32), 1.7, gain, EPS, torch.bfloat16)
        y = ops.linear_for_stream(inner, w)
        met += isinstance(y, PartialSums)
        fused = ops.scaled_add_rms_norm(x, y, 1.7, gain, EPS, torch.bfloat16)
        what = f"{T} tokens, width {d}, K {K}"
        assert float((whole[0] - fused[0]).abs().max() / whole[0].abs().max()) < 2e-6, what
        assert bool(((whole[1].float() - fused[1].float()).abs() <= 2.0**-7 * whole[1].float().abs() + 1e-30).all()), what
    assert met, "no shape ran with partial sums"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V", [(3, 24, 40), (2, 96, 20), (1, 16, 16), (4, 64, 64), (2, 160, 130), (5, 8, 3)])
def test_lightning_attention_alone(dtype, H, D, V):
    """Whole, in portions down to one token, and three requests of unequal length in one step
    with slots in another order, each against the plain recurrence; decays from 0.3 to exactly 1."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d, T = 48, 37
    g = torch.Generator().manual_seed(H * 100 + D)
    decay = [0.3, 1.0, 0.9, 0.999, 0.6][:H]
    m = dict(heads=H, dim=D, vdim=V, decay=decay)
    shapes = {"q": (H * D, d), "k": (H * D, d), "v": (H * V, d), "g": (H * V, d), "o": (d, H * V)}
    w = {"m." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in shapes.items()}
    w["m.norm"] = 1 + 0.1 * torch.randn(H * V, generator=g)
    part = build_part("mixer", PartSpec("lightning_attention", dict(m, eps=EPS), "m."), d)
    part.load(on_device(w, dtype))
    hs = [rounded(torch.randn(n, d, generator=g)) for n in (T, 5, 1)]
    refs = [plain.lightning_mixer({k: v.double() for k, v in w.items()}, "m.", m, EPS, h.double())[0].float() for h in hs]
    state = torch.zeros(6, H, D, V, device="cuda")
    view = CacheView(state={"s": state})

    def run(pieces, lens, slots):
        h = torch.cat(pieces).cuda().to(dtype)
        return part.forward(h, None, step_context(lens, [0] * len(lens), slots), view).float().cpu()

    tol = 0.05  # bfloat16: the projections, the gated output and the result are each rounded once
    check(run([hs[0]], [T], [2]), refs[0], dtype, "whole", tol)
    state.zero_()
    got, at = [], 0
    for n in (1, 2, 16, 1, 17):  # across the kernel's token tile of 16
        got.append(run([hs[0][at : at + n]], [n], [4]))
        at += n
    check(torch.cat(got), refs[0], dtype, "in portions", tol)
    assert not state[[0, 1, 2, 3, 5]].any(), "a slot other than the request's was written"
    state.zero_()
    out = run(hs, [T, 5, 1], [5, 0, 3])
    check(out, torch.cat(refs), dtype, "three requests in one step", tol)
    assert out.dtype == torch.float32


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V", [(3, 24, 40), (2, 96, 20), (2, 64, 64)])
def test_lightning_attention_in_segments(dtype, H, D, V):
    """Portions long enough to be cut into segments that run side by side: after a first portion
    that leaves a state, beside short requests in the same step, and followed by single tokens;
    segments of 64 tokens, the last one ragged; equal to the recurrence token by token."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d = 48
    g = torch.Generator().manual_seed(H + D)
    m = dict(heads=H, dim=D, vdim=V, decay=[0.97, 1.0, 0.5][:H])
    shapes = {"q": (H * D, d), "k": (H * D, d), "v": (H * V, d), "g": (H * V, d), "o": (d, H * V)}
    w = {"m." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in shapes.items()}
    w["m.norm"] = 1 + 0.1 * torch.randn(H * V, generator=g)
    part = build_part("mixer", PartSpec("lightning_attention", dict(m, eps=EPS), "m."), d)
    part.load(on_device(w, dtype))
    lens = [20 + 300 + 3, 1, 5, 256]
    hs = [rounded(torch.randn(n, d, generator=g)) for n in lens]
    refs = [plain.lightning_mixer({k: v.double() for k, v in w.items()}, "m.", m, EPS, h.double())[0].float() for h in hs]
    view = CacheView(state={"s": torch.zeros(5, H, D, V, device="cuda")})

    def run(pieces, starts, slots):
        h = torch.cat(pieces).cuda().to(dtype)
        return part.forward(h, None, step_context([len(x) for x in pieces], starts, slots), view).float().cpu()

    first = run([hs[0][:20]], [0], [3])
    both = run([hs[0][20:320], hs[1], hs[2], hs[3]], [20, 0, 0, 0], [3, 0, 4, 1])
    last = torch.cat([run([hs[0][320 + i : 321 + i]], [320 + i], [3]) for i in range(3)])
    tol = 0.05
    check(torch.cat([first, both[:300], last]), refs[0], dtype, "a long portion between a short one and single tokens", tol)
    check(both[300:301], refs[1], dtype, "one token beside it", tol)
    check(both[301:306], refs[2], dtype, "five tokens beside it", tol)
    check(both[306:], refs[3], dtype, "a portion of exactly four segments", tol)


def latent_weights(g, d, m, own):
    H, D, Rt, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    shapes = {"q": (H * (D + Rt), d), "uk": (H * D, R), "uv": (H * V, R), "g": (H, d), "o": (d, H * V)}
    if own:
        shapes["dkv"] = (R + Rt, d)
    w = {"m." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in shapes.items()}
    if own:
        w["m.dkv.norm"] = 1 + 0.1 * torch.randn(R, generator=g)
    return w


def latent_part(d, m, reads):
    from atomserve_b200.parts import PartSpec, build_part

    position = PartSpec("rotary", dict(head_dim=m["rot_dim"], theta=m["rot"]["base"], rotary_dim=m["rot"]["dims"], pairing="interleaved"))
    return build_part("mixer", PartSpec("latent_attention", dict(
        heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"],
        eps=EPS, position=position, reads_cache_of_another=reads), "m."), d)  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,Rt,dims,V,R,bs", [(5, 24, 8, 8, 16, 40, 4), (1, 32, 16, 8, 32, 64, 16), (8, 16, 4, 4, 8, 24, 8),
                                               (3, 64, 32, 32, 48, 136, 16), (40, 8, 2, 2, 8, 16, 2)])  # fmt: skip
def test_latent_attention_alone(dtype, H, D, Rt, dims, V, R, bs):
    """One sequence in portions cut inside pages, scattered over pages in no order; then a second
    mixer with other heads reading the first one's pages. The scale makes the softmax pick single
    keys, near and far."""
    from atomserve_b200.parts import CacheView

    d, T = 56, 75
    g = torch.Generator().manual_seed(H + R)
    m = dict(heads=H, dim=D, rot_dim=Rt, vdim=V, kv_rank=R, scale=2.5 / math.sqrt(D + Rt), rot=dict(base=300.0, dims=dims))
    m2 = dict(m, heads=2, dim=12, vdim=20, scale=3.0 / math.sqrt(12 + Rt))
    w, w2 = latent_weights(g, d, m, True), latent_weights(g, d, m2, False)
    part, reader = latent_part(d, m, False), latent_part(d, m2, True)
    part.load(on_device(w, dtype))
    reader.load(on_device(w2, dtype))
    h, h2 = rounded(torch.randn(T, d, generator=g)), rounded(torch.randn(T, d, generator=g))
    pos = torch.arange(T)
    wd, w2d = {k: v.double() for k, v in w.items()}, {k: v.double() for k, v in w2.items()}
    keys = plain.latent_keys(wd, "m.", m, EPS, h.double(), pos)
    ref = plain.latent_attention_mixer(wd, "m.", m, EPS, h.double(), pos, keys).float()
    ref2 = plain.latent_attention_mixer(w2d, "m.", m2, EPS, h2.double(), pos, keys).float()
    pages = -(-T // bs)
    table = torch.randperm(pages + 3, generator=g)[:pages].tolist()
    view = CacheView(pages={"latent": torch.zeros(pages + 3, 1, bs, R + Rt, device="cuda", dtype=dtype)}, block_size=bs)
    view.block_tables = torch.tensor([table], dtype=torch.int32, device="cuda")
    got, got2, at = [], [], 0
    for n in (3, 1, 2, 29, 1, 33, 6):
        view.slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(at, at + n)], dtype=torch.int32, device="cuda")
        ctx = step_context([n], [at])
        got.append(part.forward(h[at : at + n].cuda().to(dtype), None, ctx, view, True).float().cpu())
        got2.append(reader.forward(h2[at : at + n].cuda().to(dtype), None, ctx, view, False).float().cpu())
        at += n
    assert at == T
    check(torch.cat(got), ref, dtype, "own pages", 0.05)
    check(torch.cat(got2), ref2, dtype, "another mixer's pages", 0.05)


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_finds_one_far_key_among_many(dtype):
    """A long context split over key partitions, a decoded token whose query matches one key far
    back: with that key's page pointing elsewhere the output would be another value."""
    from atomserve_b200 import ops

    H, R, Rt, bs, S = 3, 40, 8, 16, 1500
    g = torch.Generator().manual_seed(5)
    keys = rounded(torch.randn(S, R + Rt, generator=g) * 0.3)
    target = [7, 700, 1499 - 16]
    q = torch.zeros(1, H, R + Rt)
    for hh, j in enumerate(target):
        q[0, hh] = keys[j] * 40  # this head's score at key j stands far above all others
    table = torch.randperm(S // bs + 1, generator=g).tolist()
    pages = torch.zeros(S // bs + 1, 1, bs, R + Rt, dtype=dtype)
    for j in range(S):
        pages[table[j // bs], 0, j % bs] = keys[j].to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    for partitions in (None, (256, 6), (1 << 30, 1)):
        out = ops.latent_attention(q.cuda(), pages.cuda(), i32([table]), i32([0, 1]), i32([S - 1]), rank=R, num_requests=1,
                                   max_context=S, scale=1.0, partitions=partitions).cpu()  # fmt: skip
        for hh, j in enumerate(target):
            assert (out[0, hh] - keys[j, :R]).abs().max() < 1e-3, f"head {hh} did not return key {j} ({partitions})"


def test_expert_selection():
    """The chosen experts and their weights against the plain rule, with and without groups, one
    and several choices, groups of one expert, every group kept."""
    from atomserve_b200 import ops

    g = torch.Generator().manual_seed(3)
    for E, top, groups, scale in ((18, 3, (3, 1), 2.2), (6, 2, (3, 2), 1.7), (4, 1, None, 1.0), (8, 3, (2, 2), 2.0),
                                  (5, 5, None, 0.5), (12, 3, (12, 4), 1.0), (64, 8, (8, 3), 1.3), (40, 32, None, 1.0)):  # fmt: skip
        z = torch.randn(33, E + 1, generator=g) * 2
        router = dict(experts=E, top=top, scale=scale)
        if groups:
            router["groups"] = dict(count=groups[0], keep=groups[1])
        want_ids, want_w = plain.route(torch.sigmoid(z[:, :E].double()), router)
        ids, weights, gate = ops.route(z.cuda(), experts=E, top=top, groups=groups[0] if groups else 1, group_top=2,
                                       keep=groups[1] if groups else 1, scale=scale, gate_col=E)  # fmt: skip
        assert torch.equal(ids.cpu().long(), want_ids), f"{E} experts, top {top}, groups {groups}"
        assert (weights.cpu().double() - want_w).abs().max() < 1e-6
        assert (gate.cpu().double() - torch.sigmoid(z[:, E].double())).abs().max() < 1e-6
        offsets, row_token, pair_row = ops.group_by_expert(ids, E)
        offsets, row_token, pair_row = offsets.cpu(), row_token.cpu(), pair_row.cpu()
        assert offsets[0] == 0 and offsets[-1] == 33 * top
        for t in range(33):
            for k in range(top):
                row = int(pair_row[t, k])
                assert row_token[row] == t and offsets[ids[t, k]] <= row < offsets[ids[t, k] + 1]


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forwards_alone(dtype):
    from atomserve_b200.parts import PartSpec, build_part

    d, T = 64, 150
    g = torch.Generator().manual_seed(9)
    h = rounded(torch.randn(T, d, generator=g))
    hd = h.cuda().to(dtype)
    # dense, both forms of the GELU
    w = {"f.up": rounded(torch.randn(100, d, generator=g) * d**-0.5), "f.down": rounded(torch.randn(d, 100, generator=g) * 0.1)}
    ff = build_part("feed_forward", PartSpec("gelu_mlp", dict(intermediate_size=100), "f."), d)
    ff.load(on_device(w, dtype))
    out = ff.forward(hd, None, None)
    assert out.dtype == torch.float32
    check(out, plain.dense_feed_forward({k: v.double() for k, v in w.items()}, "f.", h.double()).float(), dtype, "dense", 0.02)
    # routed experts of three kinds; equal inputs, so selection is the oracle's in bfloat16 too
    for E, top, groups, ff_size, limit, shared in ((6, 2, (3, 2), 48, 1.5, (32, 3.0)), (4, 1, None, 36, 0.5, None),
                                                   (15, 4, (3, 2), 72, 1.8, (24, 1.0))):  # fmt: skip
        mlp = dict(kind="moe", expert=dict(ff=ff_size, limit=limit), router=dict(experts=E, top=top, scale=1.7))
        if groups:
            mlp["router"]["groups"] = dict(count=groups[0], keep=groups[1])
        names = [f"e{e}" for e in range(E)]
        sizes = {n: ff_size for n in names}
        if shared:
            mlp["shared"] = dict(ff=shared[0], limit=shared[1])
            sizes["shared"] = shared[0]
        w = {"f.router": rounded(torch.randn(E, d, generator=g) * 0.3)}
        for n, s in sizes.items():
            w.update({f"f.{n}.gate": rounded(torch.randn(s, d, generator=g) * 0.3), f"f.{n}.up": rounded(torch.randn(s, d, generator=g) * 0.3),
                      f"f.{n}.down": rounded(torch.randn(d, s, generator=g) * 0.2)})  # fmt: skip
        if shared:
            w["f.shared.sg"] = rounded(torch.randn(1, d, generator=g) * 0.3)
        part = build_part("feed_forward", PartSpec("routed_experts", dict(
            experts=E, top=top, expert_ff=ff_size, limit=limit, groups=groups[0] if groups else 1, keep=groups[1] if groups else 1,
            scale=1.7, slope=1.702, shift=1.0, shared_ff=shared[0] if shared else None, shared_limit=shared[1] if shared else None), "f."), d)  # fmt: skip
        part.load(on_device(w, dtype))
        ref = plain.expert_feed_forward({k: v.double() for k, v in w.items()}, "f.", mlp, h.double()).float()
        for rows in (slice(0, T), slice(3, 4), slice(10, 75)):  # many tokens, one, and more than a tile of rows
            check(part.forward(hd[rows].contiguous(), None, None), ref[rows], dtype, f"{E} experts, rows {rows}", 0.02)


# ---- whole models through the step function ---------------------------------------------------

LENGTHS = {"a": [5, 49, 130, 1, 64], "b": [33, 2, 97, 40], "c": [150, 9, 70]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> (config, block size, folder, prompts, float64 logits per prompt). The
    bfloat16 models choose every allowed expert (`calm`)."""
    out = {}
    for name, (cfg, bs) in GEFILIX.items():
        for dtype in ("float32", "bfloat16"):
            c = cfg if dtype == "float32" else calm(cfg)
            w = plain.random_checkpoint(c, seed=31)
            folder = write_folder(c, w, tmp_path_factory.mktemp(f"gefilix_{name}_{dtype}"))
            ps = prompts(c, LENGTHS[name], seed=6)
            out[name, dtype] = (c, bs, folder, ps, [oracle(w, c, p) for p in ps])
    return out


def replayer(folder, dtype, bs, max_tokens, **more):
    from atomserve_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, bs, **more)


CASES = [(n, d) for n in GEFILIX for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_then_token_by_token_then_portions(models, name, dtype):
    cfg, bs, folder, ps, refs = models[name, dtype]
    rp = replayer(folder, dtype, bs, max(-(-len(p) // 64) * 64 for p in ps))
    sizes = [2, 7, 3, 16, 2, 17, 5, 31, 2, 9, 1, 33]
    for i, (p, ref) in enumerate(zip(ps, refs)):
        n = len(p)
        check(rp.step([dict(id=i, tokens=p, want=list(range(n)))], end=[i]), ref, dtype, f"{name} request {i} whole")
        head = max(n - 40, 0)
        if head:
            check(rp.step([dict(id=i, tokens=p[:head], want=[0, head - 1])], end=[]), ref[[0, head - 1]], dtype, f"{name} request {i} head")
        for j in range(head, n):
            logits = rp.step([dict(id=i, tokens=[p[j]], want=[0])], end=[i] if j == n - 1 else [])
            check(logits, ref[j : j + 1], dtype, f"{name} request {i} position {j} alone")
        at, k = 0, i
        while at < n:
            m = min(sizes[k % len(sizes)], n - at)
            k += 1
            logits = rp.step([dict(id=i, tokens=p[at : at + m], want=list(range(m)))], end=[i] if at + m == n else [])
            check(logits, ref[at : at + m], dtype, f"{name} request {i} portion {at}:{at + m}")
            at += m


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_requests_reusing_pages_and_slots(models, name, dtype):
    """Up to four live requests in four state slots, portions beside single tokens, in a pool so
    small that pages and slots freed by finished requests are taken again; every request appears
    four times, each equal to itself alone."""
    cfg, bs, folder, ps, refs = models[name, dtype]
    ps3, refs3 = ps * 4, refs * 4
    biggest = sorted((-(-len(p) // 64) * 64 for p in ps3), reverse=True)
    rp = replayer(folder, dtype, bs, sum(biggest[:4]), max_live=4)
    rng = np.random.default_rng(11)
    for entries, end in mixed_trace(ps3, rng, largest=40):
        logits = rp.step([dict(id=e["id"], tokens=e["tokens"], want=e["want"]) for e in entries], end=end)
        row = 0
        for e in entries:
            n = len(e["tokens"])
            check(logits[row : row + n], refs3[e["id"]][e["at"] : e["at"] + n], dtype, f"{name} request {e['id']} at {e['at']}")
            row += n
    assert sum(len(p) for p in ps3) > rp.cache.num_blocks * bs, "the pool was large enough to never reuse a page"
    assert len(ps3) > 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """400 tokens one by one after a short prompt: across many pages and key partitions, the
    recurrent state carried through every step."""
    for name in ("a", "c"):
        cfg, bs, folder, _, _ = models[name, dtype]
        w = plain.random_checkpoint(cfg, seed=31)
        p = prompts(cfg, [420], seed=12)[0]
        ref = oracle(w, cfg, p)
        rp = replayer(folder, dtype, bs, 448)
        rp.step([dict(id="x", tokens=p[:20], want=[])], end=[])
        for j in range(20, len(p)):
            logits = rp.step([dict(id="x", tokens=[p[j]], want=[0])], end=[])
            if j % 9 == 0 or j > 410:
                check(logits, ref[j : j + 1], dtype, f"{name} decode position {j}")


# ---- generation through the engine -----------------------------------------------------------

GREEDY = dict(temperature=0.0, ignore_eos=True)


def engine_for(folder, dtype, bs, **kw):
    from atomserve_b200.config import EngineConfig
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.weights import load_model

    _, _, model = load_model(folder, dtype, "cuda")
    config = EngineConfig(**{"block_size": bs, "num_blocks": 64, "max_model_len": 64 * bs, "max_num_seqs": 8,
                             "max_num_batched_tokens": 256, **kw})  # fmt: skip
    return create_engine(model, config, sampler_seed=0)


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_through_the_engine(models, name):
    """The engine's own entry point and scheduler: batched, in portions under a small budget, and
    with so few pages that requests are preempted and recomputed (state slots given back and
    zeroed again); float32 tokens equal the plain implementation's."""
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, folder, _, _ = models[name, "float32"]
    w = plain.random_checkpoint(cfg, seed=31)
    ps = prompts(cfg, [5, 17, 33], seed=3)
    expect = [plain.greedy_generate(w, cfg, p, 8) for p in ps]
    params = SamplingParams(max_tokens=8, **GREEDY)
    assert engine_for(folder, "float32", bs).generate(ps, params) == expect
    chunked = engine_for(folder, "float32", bs, max_num_batched_tokens=8, max_num_seqs=4)
    assert chunked.generate(ps, params) == expect
    assert chunked.num_steps > 8 + 3
    short = engine_for(folder, "float32", bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    n = bs + 8
    ps2 = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    assert short.generate(ps2, SamplingParams(max_tokens=n, **GREEDY)) == [plain.greedy_generate(w, cfg, p, n) for p in ps2]
    assert short.stats()["preemptions"] > 0 and short.stats()["kv_blocks_used"] == 0


def test_greedy_generation_in_bfloat16_picks_near_best_tokens(models):
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, folder, _, _ = models["c", "bfloat16"]
    w = plain.random_checkpoint(cfg, seed=31)
    ps = prompts(cfg, [40, 7, 90], seed=3)
    outs = engine_for(folder, "bfloat16", bs, max_num_batched_tokens=48).generate(ps, SamplingParams(max_tokens=12, **GREEDY))
    for p, out in zip(ps, outs):
        assert len(out) == 12
        ref = oracle(w, cfg, list(p) + list(out))
        spread = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
        for i, token in enumerate(out):
            row = ref[len(p) + i - 1]
            assert float(row.max() - row[token]) <= 0.15 * spread, f"token {i} lies far below the best"


def test_command_line_and_random_weights(tmp_path):
    """`python -m atomserve_b200` on a Gefilix folder written by the package's own random-weights
    writer from a configuration that round-trips through config.json."""
    import json
    import subprocess
    import sys

    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.weights.random_init import write_model_folder

    arch, config = config_from_dict(GEFILIX["b"][0])
    assert arch.name == "Gefilix" and config_from_dict(config.to_dict())[1] == config
    folder = write_model_folder(config, 3, tmp_path / "m", "bfloat16")
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Gefilix"
    done = subprocess.run([sys.executable, "-m", "atomserve_b200", str(folder), "--prompt-ids", "5,6,7", "--max-tokens", "6",
                           "--temperature", "0"], capture_output=True, text=True, timeout=600)  # fmt: skip
    assert done.returncode == 0, done.stderr[-2000:]

"""The Zogepel design on the GPU against the plain implementation: each mechanism's part alone,
then whole models through the trace replayer in every way of cutting requests into steps, then
greedy generation through the engine and its scheduler."""

import numpy as np
import pytest
import torch

import plain_zogepel as plain
from gefilix_helpers import check, prompts, write_folder
from helpers import mixed_trace
from test_engine_gpu import step_context
from tiny_zogepel import ZOGEPEL

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
EPS = 1e-5
F64 = torch.float64


def rounded(t):
    return t.bfloat16().float()


def on_device(w, dtype):
    return {k: v.cuda().to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()}


def doubles(w, prefix=""):
    return {k[len(prefix):]: v.double() for k, v in w.items() if k.startswith(prefix)}


# ---- each mechanism alone -------------------------------------------------------------------


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [72, 328, 1030])
def test_norm_on_the_sublayers_output(dtype, d):
    """x + mult * N(y) * gain * scale with the centred and the RMS norm, with and without a layer
    scale, with the sublayer's output given as two halves, and the norm alone on chosen rows."""
    from atomserve_b200 import ops
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(d)
    T = 11
    gain, scale, ga, gb = (1 + 0.1 * torch.randn(d, generator=g) for _ in range(4))
    x, y, b = torch.randn(T, d, generator=g), 3 + 2 * torch.randn(T, d, generator=g), 0.1 * torch.randn(T, d, generator=g)
    norm = build_part("norm", PartSpec("output_norm", dict(eps=EPS, mult=0.6, tensor="n", scale_tensor="s")), d)
    norm.load({"n": gain.cuda(), "s": scale.cuda()})
    norm.bind_dtype(dtype)
    stream, copy = norm.add_forward(x.cuda(), y.cuda())
    ref = x.double() + 0.6 * plain.layer_norm(y.double(), gain.double(), EPS) * scale.double()
    check(stream, ref.float(), torch.float32, "stream after a centred norm")
    assert stream.dtype == torch.float32 and copy.dtype == dtype and torch.equal(copy.float(), stream.to(dtype).float())
    joined = 0.5 * (plain.rms_unit(y.double(), EPS) * ga.double() + plain.rms_unit(b.double(), EPS) * gb.double())
    stream, _ = norm.add_forward(x.cuda(), y.cuda(), (b.cuda(), ga.cuda(), gb.cuda()))
    check(stream, (x.double() + 0.6 * plain.layer_norm(joined, gain.double(), EPS) * scale.double()).float(), torch.float32, "two halves")
    plain_rms = ops.residual_out_norm(x.cuda(), y.cuda(), gain.cuda(), EPS, dtype, mult=1.3, centred=False)[0]
    check(plain_rms, (x.double() + 1.3 * plain.rms_unit(y.double(), EPS) * gain.double()).float(), torch.float32, "RMS form, no layer scale")
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    last = norm.forward(y.cuda(), rows)
    assert last.dtype == dtype
    check(last, plain.layer_norm(y.double(), gain.double(), EPS).float()[[7, 0, 3]], dtype, "the norm alone on chosen rows", 0.01)


@pytest.mark.parametrize("M,N,K", [(1, 392, 328), (8, 8192, 2048), (33, 100, 64), (200, 1024, 512), (600, 768, 256), (2048, 4096, 1024), (1024, 5000, 2048)])
def test_squared_relu_in_the_products_epilogue(M, N, K):
    """max(x W^T, 0)^2 from the tensor-core GEMMs' epilogues (few tokens with K cut and a reduction
    kernel, single SMs, pairs of SMs, a last round cut along K) against float64, rounded once."""
    from atomserve_b200 import ops

    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * K**-0.5).bfloat16()
    got = ops.linear_relu2(x.cuda(), w.cuda())
    assert got is not None and got.dtype == torch.bfloat16
    ref = torch.relu(x.double() @ w.double().T) ** 2
    err = (got.double().cpu() - ref).abs()
    assert bool((err <= 2.0**-8 * ref.abs() + 1e-4).all()), float((err / (ref.abs() + 1e-3)).max())
    part = build_relu2_mlp(K, N, x, w)
    assert torch.equal(part, got.cpu())


def build_relu2_mlp(K, N, x, w):
    """The feed-forward part's inner activation: the fused product."""
    from atomserve_b200.parts import PartSpec, build_part

    part = build_part("feed_forward", PartSpec("activation_mlp", dict(intermediate_size=N, activation="relu2"), "f."), K)
    part.load({"f.up": w.cuda(), "f.down": torch.zeros(K, N, dtype=torch.bfloat16, device="cuda")})
    return part.inner(x.cuda()).cpu()


def test_output_norm_reading_a_products_partial_sums():
    """With few tokens the last product of a sublayer stays as the GEMM's partial sums and the
    norm's kernel adds them up: the finished product followed by the norm, up to the order in
    which a row's sums are formed (a few float32 ulps; the bfloat16 copy within one of its own)."""
    from atomserve_b200 import ops
    from atomserve_b200.ops.linear import PartialSums

    g = torch.Generator().manual_seed(4)
    met = 0
    for T, d, K in ((1, 256, 512), (5, 336, 1024), (8, 2048, 2048), (33, 256, 392)):
        inner = (torch.randn(T, K, generator=g)).bfloat16().cuda()
        w = (torch.randn(d, K, generator=g) * K**-0.5).bfloat16().cuda()
        x = torch.randn(T, d, generator=g).cuda()
        gain, scale = ((1 + 0.1 * torch.randn(d, generator=g)).cuda() for _ in range(2))
        for centred, sc in ((True, scale), (False, None)):
            whole = ops.residual_out_norm(x, ops.linear(inner, w, out_dtype=torch.float32), gain, EPS, torch.bfloat16, mult=0.6,
                                          scale=sc, centred=centred)  # fmt: skip
            y = ops.linear_for_stream(inner, w)
            met += isinstance(y, PartialSums)
            fused = ops.residual_out_norm(x, y, gain, EPS, torch.bfloat16, mult=0.6, scale=sc, centred=centred)
            what = f"{T} tokens, width {d}, K {K}, centred {centred}"
            assert float((whole[0] - fused[0]).abs().max() / whole[0].abs().max()) < 2e-6, what
            assert bool(((whole[1].float() - fused[1].float()).abs() <= 2.0**-7 * whole[1].float().abs() + 1e-30).all()), what
    assert met, "no shape ran with partial sums"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,dim,layers,layer", [(96, 12, 4, 2), (256, 16, 3, 0), (64, 1, 2, 1)])
def test_token_input_alone(dtype, d, dim, layers, layer):
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(dim)
    V, T = 50, 9
    w = {"t": rounded(torch.randn(V, layers * dim, generator=g)), "p.gate": rounded(torch.randn(dim, d, generator=g) * d**-0.5),
         "p.proj": rounded(torch.randn(d, dim, generator=g)), "p.norm": 1 + 0.1 * torch.randn(d, generator=g)}  # fmt: skip
    part = build_part("token_input", PartSpec("gated_token_slice", dict(vocab_size=V, table="t", table_width=layers * dim,
                                                                        offset=layer * dim, dim=dim, eps=EPS, mult=0.6), "p."), d)  # fmt: skip
    part.load(on_device(w, dtype))
    part.bind_dtype(dtype)
    x = rounded(torch.randn(T, d, generator=g))
    ids = torch.randint(0, V, (T,), generator=g)
    ctx = step_context([T], [0])
    ctx.token_ids = ids.to(torch.int32).cuda()
    stream, copy = part.forward(x.cuda(), x.cuda().to(dtype), ctx)
    ref = x.double() + 0.6 * plain.token_side(x.double(), ids, w["t"].double(), doubles(w, "p."), layer, dim, EPS)
    check(stream, ref.float(), dtype, "stream after the token input", 0.02)
    assert stream.dtype == torch.float32 and copy.dtype == dtype


def test_gates_and_their_running_maximum():
    """The log gates, the running maximum carried in the state across portions (starting at 0, not
    at minus infinity), and each token's decay and input weight, against the recurrence written out;
    pre-activations far beyond the cap on both sides."""
    from atomserve_b200 import ops

    g = torch.Generator().manual_seed(5)
    H, cap = 3, 6.0
    lens = [70, 1, 300]
    z = [8 * torch.randn(n, 2 * H + 1, generator=g) for n in lens]
    bi, bf = torch.randn(H, generator=g), 1 + torch.randn(H, generator=g)
    state = torch.zeros(5, H, device="cuda")
    slots = [3, 0, 4]
    got = {i: [] for i in range(3)}
    for cut in ([(0, 0, 70), (1, 0, 1), (2, 0, 17)], [(2, 17, 283)]):  # three requests in a step, then the rest of the third
        rows = torch.cat([z[i][a : a + n] for i, a, n in cut]).cuda()
        ctx = step_context([n for _, _, n in cut], [a for _, a, _ in cut], [slots[i] for i, _, _ in cut])
        out = ops.capped_gates_scan(rows, 1, 1 + H, H, bi.cuda(), bf.cuda(), cap, state, ctx.state_slots, ctx.req_q_start, len(cut))
        at = 0
        for i, _, n in cut:
            got[i].append(torch.stack([o[at : at + n].cpu() for o in out]))
            at += n
    for i, n in enumerate(lens):
        zi, zf = z[i][:, 1 : 1 + H].double() + bi.double(), z[i][:, 1 + H :].double() + bf.double()
        li = cap * torch.tanh(zi / cap)
        lf = torch.nn.functional.logsigmoid(cap * torch.tanh(zf / cap))
        top, ref = torch.zeros(H, dtype=F64), []
        for t in range(n):
            new = torch.maximum(lf[t] + top, li[t])
            ref.append(torch.stack([torch.exp(lf[t] + top - new), torch.exp(li[t] - new), new]))
            top = new
        ref = torch.stack(ref, 1)
        assert torch.allclose(torch.cat(got[i], 1).double(), ref, rtol=2e-5, atol=1e-6), f"request {i}"
        assert torch.allclose(state[slots[i]].cpu().double(), top, rtol=1e-6, atol=1e-6)
    assert not state[[1, 2]].any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V,cap", [(3, 24, 40, 6.0), (2, 96, 20, 15.0), (1, 16, 16, 2.0), (4, 64, 64, 12.0), (2, 130, 127, 8.0), (5, 8, 3, 4.0)])
def test_matrix_memory_alone(dtype, H, D, V, cap):
    """Whole, in portions down to one token, three requests of unequal length in one step with
    slots in another order, and a portion long enough to run in segments after a first one that
    leaves a state: each against the plain recurrence."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d, T = 48, 37
    g = torch.Generator().manual_seed(H * 100 + D)
    m = dict(heads=H, dim=D, vdim=V, gate_cap=cap)
    shapes = {"q": (H * D, d), "k": (H * D, d), "v": (H * V, d), "g": (H * V, d), "o": (d, H * V), "i": (H, d), "f": (H, d)}
    w = {"m." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in shapes.items()}
    w["m.i"], w["m.f"] = w["m.i"] * 3, w["m.f"] * 3  # gates that move
    w.update({"m.norm": 1 + 0.1 * torch.randn(H * V, generator=g), "m.i.b": torch.randn(H, generator=g), "m.f.b": 1 + torch.randn(H, generator=g)})
    part = build_part("mixer", PartSpec("matrix_memory", dict(m, eps=EPS), "m."), d)
    part.load(on_device(w, dtype))
    hs = [rounded(torch.randn(n, d, generator=g)) for n in (T, 5, 1, 420)]
    refs = [plain.mlstm(h.double(), doubles(w, "m."), m, EPS).float() for h in hs]
    # bfloat16: twice what rounding the projections and the gated heads does to the plain implementation
    # itself (a normaliser near its floor magnifies it), at least 0.05
    tol = 0.05
    if dtype == torch.bfloat16:
        for h, ref in zip(hs, refs):
            lossy = plain.mlstm(h.double(), doubles(w, "m."), m, EPS, stored=lambda t: t.bfloat16().double()).float()
            d_ = (lossy - ref).double()
            d_ = d_ - d_.mean(-1, keepdim=True)
            spread = (ref.double() - ref.double().mean(-1, keepdim=True)).pow(2).mean().sqrt()
            tol = max(tol, 2 * float(d_.pow(2).mean(-1).sqrt().max() / spread))
    view = CacheView(state={"s": torch.zeros(7, H, D, V, device="cuda"), "n": torch.zeros(7, H, D, device="cuda"), "top": torch.zeros(7, H, device="cuda")})

    def run(pieces, lens, slots):
        h = torch.cat(pieces).cuda().to(dtype)
        return part.forward(h, None, step_context(lens, [0] * len(lens), slots), view).float().cpu()

    check(run([hs[0]], [T], [2]), refs[0], dtype, "whole", tol)
    got, at = [], 0
    for n in (1, 2, 16, 1, 17):  # across the kernel's token tile of 16
        got.append(run([hs[0][at : at + n]], [n], [4]))
        at += n
    check(torch.cat(got), refs[0], dtype, "in portions", tol)
    for buf in view.state.values():
        assert not buf[[0, 1, 3, 5, 6]].any(), "a slot other than the request's was written"
        buf.zero_()
    out = run(hs[:3], [T, 5, 1], [5, 0, 3])
    check(out, torch.cat(refs[:3]), dtype, "three requests in one step", tol)
    assert out.dtype == torch.float32
    got = torch.cat([run([hs[3][:30]], [30], [6]), run([hs[3][30:], hs[1]], [390, 5], [6, 1])])
    ref = torch.cat([refs[3], refs[1]])
    if dtype == torch.float32:
        # 420 tokens of float32 products of decays and a quotient by the normaliser: 5e-5 of the largest value
        assert float((got.double() - ref.double()).abs().max() / ref.double().abs().max()) < 5e-5
    else:
        check(got, ref, dtype, "a long portion in segments after a short one", tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V,dims", [(3, 16, 40, 8), (1, 96, 20, 96), (5, 8, 3, 0), (2, 64, 128, 32), (2, 24, 24, 12)])
def test_retention_alone(dtype, H, D, V, dims):
    """The recurrence with rotated q and k, a scaled k, heads normed one by one without a gain and a
    SiLU gate: whole, in portions (the rotation then starts mid-sequence), two requests in a step,
    and a long portion in segments; rotations of a whole head, a part of it, and none."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d = 48
    g = torch.Generator().manual_seed(H * 10 + D)
    m = dict(heads=H, dim=D, vdim=V, decay=[0.97, 1.0, 0.5, 0.9, 0.999][:H], rot=dict(base=200.0, dims=dims))
    shapes = {"q": (H * D, d), "k": (H * D, d), "v": (H * V, d), "g": (H * V, d), "o": (d, H * V)}
    w = {"m." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in shapes.items()}
    position = PartSpec("rotary", dict(head_dim=D, theta=200.0, rotary_dim=dims)) if dims else None
    part = build_part("mixer", PartSpec("lightning_attention", dict(heads=H, dim=D, vdim=V, decay=m["decay"], eps=EPS, activation="none",
                                                                    position=position, k_scale=D**-0.5, head_norm="each", norm_gain=False,
                                                                    gate="silu"), "m."), d)  # fmt: skip
    part.load(on_device(w, dtype))
    assert [s.name for s in part.tensor_specs()] == ["m.q", "m.k", "m.v", "m.g", "m.o"]
    hs = [rounded(torch.randn(n, d, generator=g)) for n in (37, 5, 400)]
    refs = [plain.retention(h.double(), doubles(w, "m."), m, EPS, torch.arange(len(h))).float() for h in hs]
    view = CacheView(state={"s": torch.zeros(6, H, D, V, device="cuda")})

    def run(pieces, lens, starts, slots):
        h = torch.cat(pieces).cuda().to(dtype)
        return part.forward(h, None, step_context(lens, starts, slots), view).float().cpu()

    tol = 0.05
    check(run([hs[0]], [37], [0], [2]), refs[0], dtype, "whole", tol)
    got, at = [], 0
    for n in (1, 2, 16, 1, 17):
        got.append(run([hs[0][at : at + n]], [n], [at], [4]))
        at += n
    check(torch.cat(got), refs[0], dtype, "in portions", tol)
    got = [run([hs[2][:9], hs[1]], [9, 5], [0, 0], [0, 1]), run([hs[2][9:]], [391], [9], [0])]
    check(torch.cat([got[0][:9], got[1]]), refs[2], dtype, "a long portion in segments after a short one", tol)
    check(got[0][9:], refs[1], dtype, "the short request beside it", tol)


class Pages:
    """Keys and values of a few requests laid into pages through scrambled block tables."""

    def __init__(self, KV, hd, bs, dtype, blocks=64, seed=0):
        self.KV, self.hd, self.bs, self.dtype = KV, hd, bs, dtype
        self.k = torch.zeros(blocks, KV, bs, hd, device="cuda", dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.free = torch.randperm(blocks, generator=torch.Generator().manual_seed(seed)).tolist()
        self.tables = {}

    def put(self, request, k, v):
        """k, v: [T, KV, hd] of positions 0 .. T - 1."""
        table = self.tables[request] = [self.free.pop() for _ in range(-(-k.shape[0] // self.bs))]
        at = torch.arange(k.shape[0])
        block = torch.tensor(table)[at // self.bs].cuda()
        self.k[block, :, (at % self.bs).cuda()] = k.to(self.dtype).cuda()
        self.v[block, :, (at % self.bs).cuda()] = v.to(self.dtype).cuda()

    def table(self, requests):
        width = max(len(self.tables[r]) for r in requests)
        return torch.tensor([self.tables[r] + [0] * (width - len(self.tables[r])) for r in requests], dtype=torch.int32, device="cuda")


def attend(q_parts, pages, requests, lens, starts, window, scale, sink):
    from atomserve_b200 import ops

    ctx = step_context(lens, starts)
    q = torch.cat(q_parts).cuda().to(pages.dtype).contiguous()
    return ops.paged_attention(q, pages.k, pages.v, pages.table(requests), ctx.req_q_start, ctx.req_pos_start,
                               num_requests=len(lens), max_context=ctx.max_context, window=window, scale=scale,
                               host_q_lens=lens, sink=sink.cuda()).float().cpu()  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd,bs,window", [(6, 2, 24, 16, 20), (4, 4, 96, 8, 7), (8, 2, 64, 16, 100), (4, 1, 128, 16, 33), (3, 3, 40, 4, 600),
                                               (8, 2, 128, 16, 600), (4, 2, 64, 16, 650), (32, 1, 64, 16, 300)])
def test_attention_with_a_sink(dtype, H, KV, hd, bs, window):
    """Random queries and keys with sinks from far below to far above the scores: a whole prompt,
    its last tokens alone (decoding), and two requests in one step, against the plain softmax with
    the sink in its denominator. Long enough for several key partitions, in the general kernel and
    (bfloat16, heads of 64 and 128) in the tensor-core kernels, also with more query heads a kv head
    than a tile of those has rows."""
    g = torch.Generator().manual_seed(H + hd)
    T, scale = 700, 2.0 * hd**-0.5
    sink = torch.linspace(-6, 6, H)
    pages = Pages(KV, hd, bs, dtype, blocks=256)
    data = {}
    for r, n in (("a", T), ("b", 45)):
        q, k, v = (rounded(torch.randn(n, heads, hd, generator=g)) for heads in (H, KV, KV))
        pages.put(r, k, v)
        data[r] = (q, plain.windowed_sink_softmax(q.double(), k.double(), v.double(), window, scale, sink.double()).float())
    tol = 0.02
    check(attend([data["a"][0]], pages, ["a"], [T], [0], window, scale, sink).flatten(1), data["a"][1].flatten(1), dtype, "whole", tol)
    for p in (T - 1, T - 2, window, window - 1, 0):
        if p < T:
            got = attend([data["a"][0][p : p + 1]], pages, ["a"], [1], [p], window, scale, sink)
            check(got.flatten(1), data["a"][1][p : p + 1].flatten(1), dtype, f"position {p} alone", tol)
    got = attend([data["b"][0][40:], data["a"][0][300:]], pages, ["b", "a"], [5, T - 300], [40, 300], window, scale, sink)
    check(got.flatten(1), torch.cat([data["b"][1][40:], data["a"][1][300:]]).flatten(1), dtype, "two requests in one step", tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,bs,hd", [(90, 16, 32), (7, 8, 32), (33, 16, 128), (16, 16, 64), (100, 16, 128), (250, 16, 128), (290, 16, 64)])
def test_one_key_stands_out_at_the_windows_edges_and_the_sink_counts_once(dtype, window, bs, hd):
    """All keys are zero but one whose score is large; its value is e_1. For a query at position p
    the key at p - window + 1 is the last one seen and the key at p - window the first one not
    seen; also the first position, the position itself, and keys on both sides of a page border.
    With zero keys elsewhere the result is known in closed form, sink included: a sink left out,
    scaled, or counted per key partition would show. Head sizes of the general kernel and of the
    tensor-core kernels (bfloat16, 64 and 128), single tokens and portions."""
    H, KV, scale, T = 2, 1, 0.5, 300
    sink = torch.tensor([1.5, -0.5])
    q = torch.zeros(1, H, hd)
    q[:, :, 0] = 8.0  # score of the marked key: 8 * 2.5 * 0.5 = 10

    def expected(seen_marked, keys_seen):
        others = keys_seen - (1 if seen_marked else 0)
        return [(np.exp(10.0) if seen_marked else 0.0) / ((np.exp(10.0) if seen_marked else 0.0) + others + np.exp(float(s))) for s in sink]

    marks = [0, 1, bs - 1, bs, 2 * bs, T - window - 1, T - window, T - window + 1, T - 2, T - 1]
    for mark in marks:
        k = torch.zeros(T, KV, hd)
        k[mark, 0, 0] = 2.5
        v = torch.zeros(T, KV, hd)
        v[mark, 0, 1] = 1.0
        pages = Pages(KV, hd, bs, dtype, seed=mark)
        pages.put("r", k, v)
        for p in sorted({T - 1, mark, min(mark + window - 1, T - 1), min(mark + window, T - 1)}):
            seen = 0 <= p - mark < window
            want = expected(seen, min(p + 1, window))
            one = attend([q], pages, ["r"], [1], [p], window, scale, sink)[0, :, 1].tolist()
            lo = max(0, p - 40)
            many = attend([q.expand(p + 1 - lo, H, hd)], pages, ["r"], [p + 1 - lo], [lo], window, scale, sink)[-1, :, 1].tolist()
            for got in (one, many):
                assert np.allclose(got, want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-6), (mark, p, got, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_attention_part_alone(dtype):
    """The mixer by itself: whole-projection norms, values that are the unnormed keys, the gate; a
    sequence in two portions and then token by token through its pages equals the plain mixer."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d, H, KV, hd, bs, T, window = 72, 6, 2, 24, 4, 41, 9
    m = dict(heads=H, kv_heads=KV, dim=hd, vdim=hd, scale=0.45, mask=dict(size=window))
    g = torch.Generator().manual_seed(0)
    shapes = {"q": (H * hd, d), "k": (KV * hd, d), "g": (H * hd, d), "o": (d, H * hd)}
    w = {"x." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in shapes.items()}
    w.update({"x.q.norm": 1 + 0.3 * torch.randn(H * hd, generator=g), "x.k.norm": 1 + 0.3 * torch.randn(KV * hd, generator=g),
              "x.sink": 2 * torch.randn(H, generator=g)})  # fmt: skip
    part = build_part("mixer", PartSpec("sink_attention", dict(num_heads=H, num_kv_heads=KV, head_dim=hd, scale=0.45, eps=EPS,
                                                               window=window), "x."), d)  # fmt: skip
    part.load(on_device(w, dtype))
    h = rounded(3 * torch.randn(T, d, generator=g))
    ref = plain.sink_window_attention(h.double(), doubles(w, "x."), m, EPS).float()
    view = CacheView(k=torch.zeros(16, KV, bs, hd, device="cuda", dtype=dtype), block_size=bs)
    view.v = torch.zeros_like(view.k)
    table = [5, 2, 7, 0, 3, 6, 11, 9, 15, 1, 4]
    view.block_tables = torch.tensor([table], dtype=torch.int32, device="cuda")
    outs = []
    for start, n in [(0, 14), (14, 9)] + [(p, 1) for p in range(23, T)]:
        view.slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(start, start + n)], dtype=torch.int32, device="cuda")
        outs.append(part.forward(h[start : start + n].cuda().to(dtype), None, step_context([n], [start]), view))
    assert outs[0].dtype == torch.float32
    check(torch.cat(outs), ref, dtype, "portions and single tokens", 0.03)


# ---- whole models through the step function ---------------------------------------------------

LENGTHS = {"a": [5, 49, 130, 1, 64], "b": [33, 2, 97, 40], "c": [300, 9, 70], "d": [20, 3, 70], "e": [45, 2, 90]}


def oracle(cfg, w, prompt):
    return plain.forward(cfg, w, prompt).float()


def row_errors(got, ref):
    """Per position: rms of the difference (mean taken off) over the spread of the reference's logits."""
    d = got.double() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    spread = (ref.double() - ref.double().mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / spread


def allowance(cfg, w, prompt, ref):
    """What rounding alone does, per position: the error of the plain implementation itself when
    everything an engine may keep in 16 bits is rounded to bfloat16. (The design norms every
    sublayer's output, so single positions magnify rounding a lot; the engine's own rounding lands
    on the same positions, see `judge`.)"""
    return row_errors(plain.forward(cfg, w, prompt, stored=lambda t: t.bfloat16().double()), ref)


def judge(got, ref, dtype, what, lossy):
    """float32: the package's rule for float32 runs. bfloat16: no position further off than four
    times what rounding alone does there (at least 0.1 of the spread: a wrong key, window edge, sink
    or state is of the order of 1), and over eight positions or more, a mean error of at most 1.5
    times that of rounding alone (at least 0.02)."""
    if dtype in ("float32", torch.float32):
        # 5e-5 of the largest logit: where a sublayer's output is small before its norm, the norm
        # magnifies float32 rounding too (the worst position of these models reaches 2.6e-5)
        got = got.float().cpu()
        assert got.shape == ref.shape and torch.isfinite(got).all(), what
        err = float((got.double() - ref.double()).abs().max() / ref.double().abs().max())
        assert err < 5e-5, f"{what}: relative error {err:.3g}"
        return
    got = got.float().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    errors = row_errors(got, ref)
    over = errors > torch.clamp(4 * lossy, min=0.1)
    assert not over.any(), f"{what}: position {int(over.nonzero()[0])} is {float(errors[over][0]):.3g} of the spread off, rounding alone {float(lossy[over][0]):.3g}"
    if len(errors) >= 8:
        assert float(errors.mean()) <= max(0.02, 1.5 * float(lossy.mean())), f"{what}: mean error {float(errors.mean()):.3g}, rounding alone {float(lossy.mean()):.3g}"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, block size, folder, weights, prompts, float64 logits per prompt, what
    rounding alone does per prompt and position)."""
    out = {}
    for name, (cfg, bs) in ZOGEPEL.items():
        w = plain.random_checkpoint(cfg, seed=17)
        folder = write_folder(cfg, w, tmp_path_factory.mktemp(f"zogepel_{name}"))
        ps = prompts(cfg, LENGTHS[name], seed=6)
        refs = [oracle(cfg, w, p) for p in ps]
        out[name] = (cfg, bs, folder, w, ps, refs, [allowance(cfg, w, p, r) for p, r in zip(ps, refs)])
    return out


def replayer(folder, dtype, bs, max_tokens, **more):
    from atomserve_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, bs, **more)


CASES = [(n, d) for n in ZOGEPEL for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_then_token_by_token_then_portions(models, name, dtype):
    cfg, bs, folder, _, ps, refs, tols = models[name]
    rp = replayer(folder, dtype, bs, max(-(-len(p) // 64) * 64 for p in ps))
    sizes = [2, 7, 3, 16, 2, 17, 5, 31, 2, 9, 1, 33]
    for i, (p, ref, tol) in enumerate(zip(ps, refs, tols)):
        n = len(p)
        judge(rp.step([dict(id=i, tokens=p, want=list(range(n)))], end=[i]), ref, dtype, f"{name} request {i} whole", tol)
        head = max(n - 40, 0)
        if head:
            judge(rp.step([dict(id=i, tokens=p[:head], want=[0, head - 1])], end=[]), ref[[0, head - 1]], dtype, f"{name} request {i} head", tol[[0, head - 1]])
        for j in range(head, n):
            logits = rp.step([dict(id=i, tokens=[p[j]], want=[0])], end=[i] if j == n - 1 else [])
            judge(logits, ref[j : j + 1], dtype, f"{name} request {i} position {j} alone", tol[j : j + 1])
        at, k = 0, i
        while at < n:
            m = min(sizes[k % len(sizes)], n - at)
            k += 1
            logits = rp.step([dict(id=i, tokens=p[at : at + m], want=list(range(m)))], end=[i] if at + m == n else [])
            judge(logits, ref[at : at + m], dtype, f"{name} request {i} portion {at}:{at + m}", tol[at : at + m])
            at += m


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_requests_reusing_pages_and_slots(models, name, dtype):
    """Up to four live requests in four state slots, portions beside single tokens, in a pool so
    small that pages and slots freed by finished requests are taken again; every request appears
    four times, each equal to itself alone."""
    cfg, bs, folder, _, ps, refs, tols = models[name]
    ps3, refs3, tols3 = ps * 4, refs * 4, tols * 4
    biggest = sorted((-(-len(p) // 64) * 64 for p in ps3), reverse=True)
    rp = replayer(folder, dtype, bs, sum(biggest[:4]), max_live=4)
    rng = np.random.default_rng(11)
    for entries, end in mixed_trace(ps3, rng, largest=40):
        logits = rp.step([dict(id=e["id"], tokens=e["tokens"], want=e["want"]) for e in entries], end=end)
        row = 0
        for e in entries:
            n = len(e["tokens"])
            judge(logits[row : row + n], refs3[e["id"]][e["at"] : e["at"] + n], dtype, f"{name} request {e['id']} at {e['at']}",
                  tols3[e["id"]][e["at"] : e["at"] + n])
            row += n
    if rp.cache.groups:  # (a model of matrix memories alone keeps no pages, only slots)
        assert sum(len(p) for p in ps3) > rp.cache.num_blocks * bs, "the pool was large enough to never reuse a page"
    assert len(ps3) > 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """400 tokens one by one after a short prompt: the windows pass over decoded tokens and pages
    they leave behind are given back, the recurrent states are carried through every step."""
    for name in ("a", "c"):
        cfg, bs, folder, w, _, _, _ = models[name]
        p = prompts(cfg, [420], seed=12)[0]
        ref = oracle(cfg, w, p)
        tol = allowance(cfg, w, p, ref)
        rp = replayer(folder, dtype, bs, 448)
        rp.step([dict(id="x", tokens=p[:20], want=[])], end=[])
        for j in range(20, len(p)):
            logits = rp.step([dict(id="x", tokens=[p[j]], want=[0])], end=[])
            if j % 9 == 0 or j > 410:
                judge(logits, ref[j : j + 1], dtype, f"{name} decode position {j}", tol[j : j + 1])


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

    cfg, bs, folder, w, _, _, _ = models[name]
    ps = prompts(cfg, [5, 17, 33], seed=3)
    expect = [plain.greedy_generate(cfg, w, p, 8) for p in ps]
    params = SamplingParams(max_tokens=8, **GREEDY)
    assert engine_for(folder, "float32", bs).generate(ps, params) == expect
    chunked = engine_for(folder, "float32", bs, max_num_batched_tokens=8, max_num_seqs=4)
    assert chunked.generate(ps, params) == expect
    assert chunked.num_steps > 8 + 3
    short = engine_for(folder, "float32", bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    n = bs + 8
    ps2 = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    assert short.generate(ps2, SamplingParams(max_tokens=n, **GREEDY)) == [plain.greedy_generate(cfg, w, p, n) for p in ps2]
    assert short.stats()["kv_blocks_used"] == 0


def test_greedy_generation_in_bfloat16_picks_near_best_tokens(models):
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, folder, w, _, _, _ = models["c"]
    ps = prompts(cfg, [40, 7, 90], seed=3)
    outs = engine_for(folder, "bfloat16", bs, max_num_batched_tokens=48).generate(ps, SamplingParams(max_tokens=12, **GREEDY))
    for p, out in zip(ps, outs):
        assert len(out) == 12
        ref = oracle(cfg, w, list(p) + list(out))
        spread = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
        for i, token in enumerate(out):
            row = ref[len(p) + i - 1]
            assert float(row.max() - row[token]) <= 0.15 * spread, f"token {i} lies far below the best"


def test_command_line_and_random_weights(tmp_path):
    """`python -m atomserve_b200` on a Zogepel folder written by the package's own random-weights
    writer from a configuration that round-trips through config.json."""
    import json
    import subprocess
    import sys

    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.weights.random_init import write_model_folder

    arch, config = config_from_dict(ZOGEPEL["b"][0])
    folder = write_model_folder(config, 3, tmp_path / "m", "bfloat16")
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Zogepel"
    done = subprocess.run([sys.executable, "-m", "atomserve_b200", str(folder), "--prompt-ids", "5,6,7", "--max-tokens", "6",
                           "--temperature", "0"], capture_output=True, text=True, timeout=600)  # fmt: skip
    assert done.returncode == 0, done.stderr[-2000:]

"""Each mechanism of the Numuzen design alone: the kernels against the plain functions of
tests/plain_numuzen.py, at sizes of their own, with inputs designed so that a fault shows (one far key
among hundreds, keys just inside and just outside the window, keys at a page's border, stale pages full
of NaN, a sink that matters, a state that must carry, experts whose scores lie apart)."""
import math

import pytest
import torch

import plain_numuzen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().double(), want.double()
    assert torch.isfinite(got).all(), f"{what}: not finite"
    err = (got - want).abs().max()
    assert err <= tol * want.abs().max(), f"{what}: {err:.3e} > {tol:.1e} * {want.abs().max():.3f}"


# ------------------------------------------------------------------ norms
@pytest.mark.parametrize("width", [64, 100, 1030])
def test_norm_with_a_weight_around_zero_before_and_behind_a_sub_layer(width):
    from torchlet_b200 import ops
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import NORMS, build_part

    w = rand(width, seed=1, scale=0.3)
    norm = build_part(NORMS, PartSpec("rms_norm", {"size": width, "eps": 1e-5, "weight_name": "", "weight_offset": 1.0}))
    norm.load({"n": w}, "n", DEV, torch.float32)
    close(norm.weight, 1.0 + w, 1e-7, "the weight as applied")
    x = rand(7, width, seed=2, scale=4.0)
    out = torch.empty(7, width, device=DEV)
    ops.rms_norm(x.to(DEV), norm.weight, 1e-5, out)
    close(out, plain.offset_norm(x.double(), w.double(), 1e-5), 1e-5, "before")
    acc = rand(7, width, seed=3)
    got = acc.to(DEV)
    ops.rms_scaled_add(got, x.to(DEV), norm.weight, 1.0, 1e-5)
    close(got, acc.double() + plain.offset_norm(x.double(), w.double(), 1e-5), 1e-5, "behind")


# ------------------------------------------------------- gated linear attention
@pytest.mark.parametrize("H,D,V,rank,tau", [(3, 12, 20, 6, 4.0), (1, 40, 8, 3, 1.0), (2, 64, 64, 16, 16.0),
                                            (1, 128, 32, 8, 8.0), (2, 10, 6, 5, 2.0), (1, 256, 72, 4, 64.0)])
def test_gla_kernels_carry_the_state(H, D, V, rank, tau):
    """decay, scan, finish against the plain recurrence: a sequence in three portions (the state
    is carried in the slot), a second request in another slot in the same launch, a padding lane,
    and the first slot used again from zero."""
    from torchlet_b200 import ops

    T, slots = 57, 3
    width = 2 * H * D + 2 * H * V + rank
    proj = rand(T, width, seed=4, scale=0.7)
    proj[:, 2 * H * D + 2 * H * V:] *= 2.0
    a2 = rand(H * D, rank, seed=5, scale=0.8)
    bias = rand(H * D, seed=6) + 1.5
    weight = 1.0 + rand(V, seed=7, scale=0.2)
    low = proj[:, -rank:].double()
    a = torch.sigmoid(low @ a2.double().T + bias.double()).pow(1.0 / tau).view(T, H, D)
    q = proj[:, :H * D].double().view(T, H, D) / math.sqrt(D)
    k = proj[:, H * D:2 * H * D].double().view(T, H, D)
    v = proj[:, 2 * H * D:2 * H * D + H * V].double().view(T, H, V)
    g = proj[:, 2 * H * D + H * V:2 * H * D + 2 * H * V].double()

    def plain_run(first, last):
        heads = [plain.linear_recurrence(q[first:last, h], k[first:last, h], v[first:last, h], a[first:last, h])[0] for h in range(H)]
        return torch.cat(heads, dim=1)

    def plain_finish(o, rows):
        o = plain.unit_rms(o.view(-1, H, V), 1e-5) * weight.double()
        return o.reshape(-1, H * V) * (g[rows] * torch.sigmoid(g[rows]))

    dproj = proj.to(DEV)
    decay = torch.empty(T, H * D, device=DEV)
    ops.gla_decay(dproj, 2 * H * D + 2 * H * V, a2.t().contiguous().to(DEV), bias.to(DEV), decay, rank, tau)
    close(decay, a.view(T, H * D), 2e-6, "decay")
    state = torch.full((slots, H, D, V), float("nan"), device=DEV)
    state[0].zero_()
    state[2].zero_()
    out = torch.full((T, H * V), float("nan"), device=DEV)
    # launch 1: request A (slot 2) tokens 0..19, a padding lane (one token), request B (slot 0) tokens 40..56
    rows1 = list(range(0, 20)) + [20] + list(range(40, 57))
    sub = dproj[rows1].contiguous()
    dsub = decay[rows1].contiguous()
    o1 = torch.full((len(rows1), H * V), float("nan"), device=DEV)
    ind = torch.tensor([0, 20, 21, 38], dtype=torch.int32, device=DEV)
    sl = torch.tensor([2, -1, 0], dtype=torch.int32, device=DEV)
    ops.gla_scan(sub, dsub, ind, sl, state, o1, 3, H, D, V, D ** -0.5)
    close(o1[:20], plain_run(0, 20), 2e-5, "A, first portion")
    assert torch.equal(o1[20], torch.zeros(H * V, device=DEV)), "a padding lane writes zeros"
    close(o1[21:], plain_run(40, 57), 2e-5, "B")
    assert torch.isnan(state[1]).all(), "a slot nobody owns is not touched"
    # launches 2 and 3: A goes on in portions of 2 and 18 tokens
    for first, last in ((20, 22), (22, 40)):
        o = torch.empty(last - first, H * V, device=DEV)
        ops.gla_scan(dproj[first:last], decay[first:last], torch.tensor([0, last - first], dtype=torch.int32, device=DEV),
                     torch.tensor([2], dtype=torch.int32, device=DEV), state, o, 1, H, D, V, D ** -0.5)
        out[first:last] = o
    close(out[20:40], plain_run(0, 40)[20:], 2e-5, "A, carried")
    # slot 0 again, zeroed as at admission: B's state must not show
    state[0].zero_()
    o = torch.empty(9, H * V, device=DEV)
    ops.gla_scan(dproj[:9], decay[:9], torch.tensor([0, 9], dtype=torch.int32, device=DEV),
                 torch.tensor([0], dtype=torch.int32, device=DEV), state, o, 1, H, D, V, D ** -0.5)
    close(o, plain_run(0, 9), 2e-5, "a slot used again")
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        fin = torch.empty(9, H * V, device=DEV, dtype=dtype)
        ops.gla_finish(o, dproj[:9], 2 * H * D + H * V, weight.to(DEV), fin, H, V, 1e-5)
        close(fin, plain_finish(plain_run(0, 9), slice(0, 9)), tol, "finish")


def test_gla_state_remembers_a_token_far_back():
    """Decay close to one in one channel: a key written 600 tokens earlier still answers its query."""
    from torchlet_b200 import ops

    H, D, V, T = 1, 16, 8, 640
    proj = torch.zeros(T, 2 * D + 2 * V + 1)
    proj[30, D + 5] = 3.0  # k of token 30, channel 5
    proj[30, 2 * D:2 * D + V] = torch.arange(1, V + 1).float()  # its value
    proj[635, 5] = 2.0  # q of token 635 asks for channel 5
    decay = torch.full((T, D), 0.5)
    decay[:, 5] = 0.9995
    state = torch.zeros(1, H, D, V, device=DEV)
    out = torch.empty(T, V, device=DEV)
    ind = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ops.gla_scan(proj.to(DEV), decay.to(DEV), ind, torch.zeros(1, dtype=torch.int32, device=DEV), state, out, 1, H, D, V, 1.0)
    want = 2.0 * 3.0 * 0.9995 ** 605 * torch.arange(1, V + 1).double()
    close(out[635], want, 1e-4, "the far token")
    assert out[29].abs().max() == 0 and out[634].abs().max() == 0


# ------------------------------------------------------------ attention
def _paged(k, v, page_size, dtype, seed=0, extra_pages=5):
    """k, v [T, G, d] into a pool whose other pages are NaN, pages handed out in a scrambled order."""
    T, G, d = k.shape
    used = -(-T // page_size)
    total = used + extra_pages + 1
    order = torch.randperm(total - 1, generator=torch.Generator().manual_seed(seed))[:used] + 1
    pages = torch.full((total, 2, G, page_size, d), float("nan"), dtype=dtype)
    for t in range(T):
        page, at = int(order[t // page_size]), t % page_size
        pages[page, 0, :, at] = k[t].to(dtype)
        pages[page, 1, :, at] = v[t].to(dtype)
    return pages.to(DEV), order.to(torch.int32).view(1, -1).to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,page_size", [(40, 16), (16, 16), (17, 8), (1, 8), (None, 32), (300, 16)])
@pytest.mark.parametrize("softcap,sink", [(None, True), (8.0, True), (8.0, False)])
def test_attention_with_cap_sink_and_window_on_designed_keys(dtype, window, page_size, softcap, sink):
    """Queries at the end of 700 keys.  Keys are weak except three that are made to stand out: the one
    JUST INSIDE the window, the one JUST OUTSIDE it (which must not be seen) and one far back (seen only
    without a window).  Values name their position, so a key that is off by one shows."""
    from torchlet_b200 import ops

    H, G, d, T, scale = 4, 2, 24, 700, 0.3
    td = TORCH[dtype]
    k = rand(T, G, d, seed=8, scale=0.05)
    v = rand(T, G, d, seed=9, scale=0.1)
    v[:, :, 0] = torch.arange(T).float().view(T, 1) / T
    q = rand(T, H, d, seed=10, scale=0.05)
    last = T - 1
    marks = [200] + ([last - window + 1, last - window] if window and window <= last else [])
    for j, at in enumerate(m for m in marks if m >= 0):
        k[at, :, 3 + j] = 6.0
        q[last, :, 3 + j] = 5.0
    k, v, q = k.to(td).float(), v.to(td).float(), q.to(td).float()
    want = torch.stack([plain.sink_softmax_attention(q[:, h].double(), k[:, h // 2].double(), v[:, h // 2].double(), scale,
                                                     softcap, window) for h in range(H)], dim=1)
    if not sink:  # the plain function always has the sink: take it out again
        for h in range(H):
            for i in range(T):
                first = 0 if not window else max(0, i - window + 1)
                s = (k[first:i + 1, h // 2].double() @ q[i, h].double()) * scale
                s = softcap * torch.tanh(s / softcap) if softcap else s
                want[i, h] = torch.softmax(s, 0) @ v[first:i + 1, h // 2].double()
    pages, table = _paged(k, v, page_size, td, seed=page_size)
    rows = [0, 1, 2, 15, 16, 17, 39, 40, 41, 255, 256, 698, 699]  # the first tokens, page and window edges, the end
    rows = [r for r in rows if r < T]
    qd = q[rows].reshape(len(rows), H * d).to(td).to(DEV)
    out = torch.full((len(rows), H * d), float("nan"), dtype=td, device=DEV)
    pos = torch.tensor(rows, dtype=torch.int32, device=DEV)
    req = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
    ops.attention_generic(qd, H * d, pages, table, req, pos, out, len(rows), H, G, d, page_size, window, scale,
                          softcap=softcap, sink=sink)
    close(out.view(len(rows), H, d), want[rows], 2e-5 if dtype == "float32" else 2e-2, "attention")


@pytest.mark.parametrize("d,H,G", [(64, 4, 1), (128, 6, 2), (64, 2, 2)])
@pytest.mark.parametrize("window,page_size", [(150, 16), (70, 16), (64, 8), (None, 16), (1, 16)])
@pytest.mark.parametrize("softcap,sink,gated", [(20.0, True, True), (None, True, False), (30.0, False, False)])
def test_tensor_core_attention_with_cap_sink_gate_equals_the_plain_kernel(d, H, G, window, page_size, softcap, sink, gated):
    """The mma.sync kernel (64-row tiles for a prompt portion, 16-row tiles with 1, 3 and 20 key splits for a
    single token, merged inside the kernel and by the second kernel) and the tcgen05 kernel (a prompt portion,
    whole and with key splits) against the one-warp-a-row kernel on the same pages, with two designed keys at
    the window's edge."""
    from torchlet_b200 import ops

    T, scale, g = 700, d ** -0.5, H // G
    td = torch.bfloat16
    k = rand(T, G, d, seed=21, scale=0.5)
    v = rand(T, G, d, seed=22, scale=0.5)
    q = rand(T, H, d, seed=23, scale=0.5)
    last = T - 1
    if window and window > 1:
        k[last - window + 1, :, 5] = 9.0
        k[last - window, :, 6] = 9.0
        q[last, :, 5:7] = 6.0
    pages, table = _paged(k, v, page_size, td, seed=d + page_size)
    gate = rand(T, H * d + 3, seed=24, scale=2.0).to(DEV) if gated else None
    gate_view = gate[:, 3:] if gated else None
    qd = q.reshape(T, H * d).to(td).to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(T, dtype=torch.int32, device=DEV)
    want = torch.empty(T, H * d, dtype=td, device=DEV)
    ops.attention_generic(qd, H * d, pages, table, zeros, pos, want, T, H, G, d, page_size, window, scale, softcap=softcap,
                          sink=sink, gate=gate_view)
    # the whole prompt as one portion, 64 packed rows a tile
    rows = torch.arange(0, T * g, 64, dtype=torch.int32, device=DEV)
    indptr = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    before = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = torch.full((T, H * d), float("nan"), dtype=td, device=DEV)
    ops.attention_mma(qd, pages, table, indptr, before, torch.zeros_like(rows), rows, rows.numel(), got, T, H, G, d, page_size,
                      window, scale, rows16=False, softcap=softcap, sink=sink, gate=gate_view)
    close(got, want.float().cpu(), 2e-2, "prompt portion")
    # the same on the tcgen05 kernel: whole, with the keys split over three CTAs, and with the merge deferred
    if ops.attention_tc_supported(d, g, page_size):
        per = ops.attention_tc_rows(g)
        rows = torch.arange(0, T * g, per, dtype=torch.int32, device=DEV)
        for splits, defer in ((1, False), (3, False), (2, True)):
            got = torch.full((T, H * d), float("nan"), dtype=td, device=DEV)
            merge = ops.attention_tc(qd, pages, table, indptr, before, torch.zeros_like(rows), rows, rows.numel(), got, H, G, d,
                                     page_size, window, scale, splits=splits, token_req=zeros, defer_merge=defer,
                                     softcap=softcap, sink=sink, gate=gate_view)
            if defer:
                merge()
            close(got, want.float().cpu(), 2e-2, f"prompt portion on tcgen05, {splits} key splits")
        ops.raise_on_wait_errors()
    # the last token alone, behind 699 cached ones
    indptr = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    before = torch.tensor([last], dtype=torch.int32, device=DEV)
    for splits in (1, 3, 20):
        one = torch.full((1, H * d), float("nan"), dtype=td, device=DEV)
        ops.attention_mma(qd[last:], pages, table, indptr, before, None, None, 1, one, 1, H, G, d, page_size, window, scale,
                          rows16=True, splits=splits, softcap=softcap, sink=sink,
                          gate=gate_view[last:] if gated else None)
        close(one, want[last:].float().cpu(), 2e-2, f"single token, {splits} key splits")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_output_gate(dtype):
    from torchlet_b200 import ops

    H, G, d, T = 2, 1, 16, 9
    td = TORCH[dtype]
    k, v, q = (rand(T, n, d, seed=s).to(td).float() for n, s in ((G, 1), (G, 2), (H, 3)))
    gate = rand(T, 7 + H * d, seed=4, scale=2.0)
    want = torch.stack([plain.sink_softmax_attention(q[:, h].double(), k[:, 0].double(), v[:, 0].double(), 0.25, None, None)
                        for h in range(H)], dim=1).reshape(T, H * d) * torch.sigmoid(gate[:, 7:].double())
    pages, table = _paged(k, v, 4, td)
    out = torch.empty(T, H * d, dtype=td, device=DEV)
    ops.attention_generic(q.reshape(T, H * d).to(td).to(DEV), H * d, pages, table, torch.zeros(T, dtype=torch.int32, device=DEV),
                          torch.arange(T, dtype=torch.int32, device=DEV), out, T, H, G, d, 4, None, 0.25, sink=True,
                          gate=gate.to(DEV)[:, 7:])
    close(out, want, 2e-5 if dtype == "float32" else 2e-2, "gated output")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dims,scaling", [(4, 2, 24, 8, True), (2, 2, 16, 16, False), (3, 1, 40, 2, True),
                                                (8, 1, 128, 32, True), (2, 1, 8, 0, False)])
def test_norm_over_the_whole_projection_rotation_and_cache_write(dtype, H, G, d, dims, scaling):
    """q and k normed over ALL heads at once (a head with large entries lowers the others), the first
    ``dims`` entries rotated by positions that start far into the sequence, the value = the key as projected."""
    from torchlet_b200 import ops
    from torchlet_b200.parts.rotary import scaled_frequencies

    T, page_size, start = 11, 4, 1234
    td = TORCH[dtype]
    rot = None
    if dims:
        rot = {"dims": dims, "base": 3000.0}
        if scaling:
            rot["scaling"] = {"factor": 3.0, "original": 40, "fast": 6.0, "slow": 1.5}
    proj = rand(T, H * d + G * d + 5, seed=11, scale=1.5)
    proj[:, :d] *= 9.0  # one head dominates the root mean square of the whole q
    wq, wk = 1.0 + rand(H * d, seed=12, scale=0.2), 1.0 + rand(G * d, seed=13, scale=0.2)
    q_want = plain.unit_rms(proj[:, :H * d].double(), 1e-5) * wq.double()
    k_want = plain.unit_rms(proj[:, H * d:H * d + G * d].double(), 1e-5) * wk.double()
    q_want = plain.rotate_heads(q_want.view(T, H, d), rot, start)
    k_want = plain.rotate_heads(k_want.view(T, G, d), rot, start)
    inv_freq, magnitude = (None, 1.0)
    if dims:
        freq, magnitude = scaled_frequencies(dims, rot["base"], rot.get("scaling"))
        want_freq, want_mag = plain.rotation_frequencies(rot)
        assert torch.allclose(freq, want_freq, rtol=1e-12) and abs(magnitude - want_mag) < 1e-12
        inv_freq = freq.float().to(DEV)
    pages = torch.full((9, 2, G, page_size, d), float("nan"), dtype=td, device=DEV)
    table = torch.zeros(1, (start + T) // page_size + 1, dtype=torch.int32, device=DEV)
    first_page = start // page_size
    table[0, first_page:first_page + 4] = torch.tensor([5, 2, 7, 3], dtype=torch.int32)
    q_out = torch.empty(T, H * d, dtype=td, device=DEV)
    pos = torch.arange(start, start + T, dtype=torch.int32, device=DEV)
    ops.normed_qk_store(proj.to(DEV), wq.to(DEV), wk.to(DEV), inv_freq, magnitude, 1e-5, pos,
                        torch.zeros(T, dtype=torch.int32, device=DEV), table, pages, page_size, q_out, H, G, d, dims, H * d)
    tol = 3e-4 if dtype == "float32" else 2e-2  # the angle of position 1,244 in float32
    close(q_out.view(T, H, d), q_want, tol, "q")
    for t in range(T):
        p = start + t
        page = int(table[0, p // page_size])
        close(pages[page, 0, :, p % page_size], k_want[t], tol, f"key of token {t}")
        close(pages[page, 1, :, p % page_size], proj[t, H * d:H * d + G * d].view(G, d), 1e-7 if dtype == "float32" else 1e-2, "value")
    assert torch.isnan(pages[[0, 1, 4, 6, 8]]).all(), "pages of others are not touched"


# -------------------------------------------------------------- experts
def _moe_weights(E, width, ff, seed):
    w = {"router": rand(E, width, seed=seed, scale=0.08)}
    for e in range(E):
        w[f"e{e}.gate"] = rand(ff, width, seed=seed + 10 + e, scale=0.3).to(torch.bfloat16).float()
        w[f"e{e}.up"] = rand(ff, width, seed=seed + 40 + e, scale=0.3).to(torch.bfloat16).float()
        w[f"e{e}.down"] = rand(width, ff, seed=seed + 70 + e, scale=0.3).to(torch.bfloat16).float()
    w["router"] = w["router"].to(torch.bfloat16).float()
    return w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,width,ff,tokens", [(5, 2, 96, 40, 150), (1, 1, 64, 24, 7), (3, 3, 64, 24, 33),
                                                   (8, 1, 72, 100, 300), (16, 4, 128, 64, 1), (6, 2, 50, 21, 70),
                                                   (4, 2, 128, 64, 500), (7, 3, 256, 320, 900), (32, 1, 64, 48, 20)])
def test_routed_feed_forward_on_given_inputs(dtype, E, top, width, ff, tokens):
    """The whole part on inputs that BOTH sides hold exactly (rounded to the engine's type first), so the
    choice of experts is the same unless two scores tie; the limit is low enough to clamp many entries."""
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import FEED_FORWARDS, build_part

    td = TORCH[dtype]
    limit = 0.9
    w = _moe_weights(E, width, ff, seed=E)
    x = rand(tokens, width, seed=20, scale=1.2).to(td).float()
    scores = torch.sigmoid(x.double() @ w["router"].double().T)
    ranked = scores.sort(dim=1, descending=True).values
    if top < E:
        x = x[(ranked[:, top - 1] - ranked[:, top]) > 1e-4]  # no close calls
        tokens = x.shape[0]
        scores = torch.sigmoid(x.double() @ w["router"].double().T)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}}
    want = plain.routed_feed_forward(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", mlp)
    part = build_part(FEED_FORWARDS, PartSpec("routed_clamped_glu", {
        "hidden_size": width, "intermediate_size": ff, "limit": limit, "alpha": 1.702, "num_experts": E, "top_k": top,
        "score": "sigmoid", "renormalize": False, "weight_on": "input"}))
    part.load({"m." + k: v for k, v in w.items()}, "m.", DEV, td)

    class Ctx:
        dtype = td
        token_capacity = 64  # smaller than the step: the scratch must grow with it

        def __init__(self):
            self.buffers = {}

        def buffer(self, name, shape, dt):
            key = (name, tuple(shape[1:]), dt)
            if key not in self.buffers or self.buffers[key].shape[0] < shape[0]:
                self.buffers[key] = torch.full(shape, float("nan") if dt != torch.int32 else -7, dtype=dt, device=DEV)
            return self.buffers[key][:shape[0]]

    ctx = Ctx()
    acc = torch.zeros(tokens, width, device=DEV)
    part.forward(ctx, x.to(td).to(DEV), acc)
    tol = 2e-5 if dtype == "float32" else 3e-2
    close(acc, want, tol, "routed feed-forward")
    choice = ctx.buffers[("moe.choice", (top,), torch.int32)][:tokens].cpu()
    order = torch.argsort(scores, dim=1, descending=True, stable=True)[:, :top]
    assert torch.equal(choice.long(), order), "the chosen experts, best first"
    again = torch.zeros(tokens, width, device=DEV)  # a second pass over the same scratch gives the same numbers
    part.forward(ctx, x.to(td).to(DEV), again)
    assert torch.equal(acc, again)


def test_router_options_and_ties():
    """Equal scores: the lower index wins.  Softmax scores renormalized over the chosen ones; the weight on
    the expert's OUTPUT."""
    from torchlet_b200 import ops

    x = torch.zeros(3, 8)
    x[1, 0] = 1.0
    x[2, 1] = 1.0
    router = torch.zeros(6, 8)
    router[:, 0] = torch.tensor([0.0, 2.0, 2.0, -1.0, 2.0, 0.5])
    router[:, 1] = torch.tensor([1.0, 1.0, 3.0, 3.0, 0.0, 3.0])
    choice = torch.empty(3, 3, dtype=torch.int32, device=DEV)
    weight = torch.empty(3, 3, device=DEV)
    ops.moe_route(x.to(DEV), router.to(DEV), choice, weight)
    assert choice.cpu().tolist() == [[0, 1, 2], [1, 2, 4], [2, 3, 5]]
    close(weight[1], torch.sigmoid(torch.tensor([2.0, 2.0, 2.0])), 1e-6)
    ops.moe_route(x.to(DEV), router.to(DEV), choice, weight, softmax_scores=True, renormalize=True)
    assert choice.cpu().tolist() == [[0, 1, 2], [1, 2, 4], [2, 3, 5]]
    close(weight, torch.full((3, 3), 1 / 3), 1e-6, "renormalized")
    ops.moe_route(x.to(DEV), router.to(DEV), choice, weight, softmax_scores=True)
    z = router[:, 0].double()
    close(weight[1], torch.softmax(z, 0)[[1, 2, 4]], 1e-6, "softmax scores")

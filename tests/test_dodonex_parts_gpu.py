"""Each mechanism of the Dodonex design alone: the kernels against the plain functions of
tests/plain_dodonex.py, at sizes of their own, with inputs designed so that a fault shows (one far
key among hundreds, a key at a page's border, stale pages full of NaN, a state that must carry)."""
import math

import pytest
import torch

import plain_dodonex as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("width,groups", [(96, 3), (64, 1), (120, 5), (4096, 4), (70, 7)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_grouped_rms_norm(width, groups, out_dtype):
    from torchlet_b200 import ops

    x = rand(9, width, seed=1, scale=3.0)
    x[:, :width // groups] *= 50.0  # a part with a scale of its own: one norm over the row would show
    w = 1.0 + rand(width, seed=2, scale=0.2)
    want = plain.group_rms_norm(x.double(), w.double(), 1e-5, groups)
    out = torch.empty(9, width, device=DEV, dtype=out_dtype)
    ops.rms_norm(x.to(DEV), w.to(DEV), 1e-5, out, None, groups)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert (out.cpu().double() - want).abs().max() <= tol * want.abs().max()
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    some = torch.empty(3, width, device=DEV, dtype=out_dtype)
    ops.rms_norm(x.to(DEV), w.to(DEV), 1e-5, some, rows, groups)
    assert torch.equal(some, out[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_glu_on_both_sides_of_the_limit(dtype):
    from torchlet_b200 import ops

    inter, limit = 52, 1.3
    gu = rand(11, 2 * inter, seed=3, scale=2.0).to(dtype)  # many values beyond the limit on either side
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    out = torch.empty(11, inter, device=DEV, dtype=dtype)
    ops.clamped_glu(gu.to(DEV), out, limit, 1.702)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert (out.cpu().double() - want).abs().max() <= tol * want.abs().max()
    assert (gu[:, :inter] < -limit).any() and (gu[:, :inter] > limit).any()  # the gate is clamped from above only


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_token_embedding_part(dtype):
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import TOKEN_INPUTS, build_part

    W, dim, V, layers, layer, m, eps = 72, 12, 50, 3, 1, 0.7, 1e-5
    w = {"side.embed": rand(V, dim * layers, seed=4).bfloat16().float(),
         f"l{layer}.side.gate": rand(dim, W, seed=5, scale=0.3).bfloat16().float(),
         f"l{layer}.side.proj": rand(W, dim, seed=6, scale=0.3).bfloat16().float(),
         f"l{layer}.side.norm": (1 + rand(W, seed=7, scale=0.1)).bfloat16().float()}
    part = build_part(TOKEN_INPUTS, PartSpec("gated_token_embedding", {
        "hidden_size": W, "dim": dim, "eps": eps, "vocab_size": V, "table_name": "side.embed",
        "table_width": dim * layers, "offset": layer * dim}))
    torch_dtype = getattr(torch, dtype)
    part.load(w, f"l{layer}.side.", DEV, torch_dtype)
    ids = torch.randint(0, V, (13,), generator=torch.Generator().manual_seed(8))
    x = rand(13, W, seed=9, scale=2.0)
    cfg = {"token_side": {"dim": dim}, "norm": {"eps": eps}}
    want = x.double() + m * plain.token_side(x.double(), ids, {k: v.double() for k, v in w.items()}, layer, cfg)

    class Ctx:
        tokens = ids.to(DEV, torch.int32)

        def __init__(self):
            self.dtype = torch_dtype

        def buffer(self, name, shape, dt):
            return torch.empty(shape, device=DEV, dtype=dt)

    acc = x.to(DEV)
    part.forward(Ctx(), acc, m)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert (acc.cpu().double() - want).abs().max() <= tol * want.abs().max()


def delta_weights(W, H, D, rank, seed):
    size = H * D
    names = {"r": (size, W), "k": (size, W), "v": (size, W), "g": (size, W), "a": (size, W), "a.b": (size,),
             "w1": (rank, W), "w2": (size, rank), "w0": (size,), "norm": (size,), "o": (W, size)}
    out = {}
    for i, (name, shape) in enumerate(names.items()):
        t = rand(*shape, seed=seed + i, scale=1.0 if len(shape) == 1 else 1.5 / math.sqrt(shape[-1]))
        out["m." + name] = (1 + 0.1 * t if name == "norm" else t).bfloat16().float()
    return out


@pytest.mark.parametrize("H,D,rank", [(2, 24, 5), (1, 64, 16), (3, 40, 7), (2, 100, 4), (1, 16, 2), (1, 200, 3), (1, 256, 8)])
def test_delta_rule_kernels_carry_the_state(H, D, rank):
    """prepare, scan and finish against the plain recurrence: a sequence in three portions (the
    state must carry), beside another request; then the first slot is used again from zero."""
    from torchlet_b200 import ops

    W, size, eps = 48, H * D, 1e-5
    w = delta_weights(W, H, D, rank, seed=10 * H + D)
    mixer = {"heads": H, "dim": D}
    hs = [rand(n, W, seed=30 + i) for i, n in enumerate((37, 9, 21))]
    fused = torch.cat([w["m." + n] for n in ("r", "k", "v", "g", "a", "w1")]).to(DEV)
    f32 = lambda name: w["m." + name].to(DEV)
    state = torch.full((3, H, D, D), float("nan"), device=DEV)  # a slot is zeroed at admission, not before

    def run(parts):  # parts: list of (slot, h rows); one step
        rows = torch.cat([h for _, h in parts]).to(DEV)
        proj = rows @ fused.T
        T = rows.shape[0]
        gates = torch.empty(T, H * 3 * D, device=DEV)
        ops.delta_prepare(proj, f32("w2").t().contiguous(), f32("w0"), f32("a.b"), gates, H, D, rank)
        indptr = torch.tensor([0] + list(torch.tensor([h.shape[0] for _, h in parts]).cumsum(0)), dtype=torch.int32,
                              device=DEV)
        slots = torch.tensor([s for s, _ in parts], dtype=torch.int32, device=DEV)
        o = torch.empty(T, size, device=DEV)
        ops.delta_scan(proj, gates, indptr, slots, state, o, len(parts), H, D)
        out = torch.empty(T, size, device=DEV)
        ops.delta_finish(o, proj, f32("norm"), out, H, D, eps)
        return (out @ f32("o").T).cpu()

    wd = {k: v.double() for k, v in w.items()}
    want = [plain.general_delta(h.double(), wd, "m.", mixer, eps)[0] for h in hs]
    state[2].zero_(); state[0].zero_()
    a = run([(2, hs[0][:5]), (0, hs[1])])          # two requests of unequal length in one step
    b = run([(2, hs[0][5:7])])                     # a portion of two tokens
    c = run([(-1, hs[1][:1]), (2, hs[0][7:])])     # beside a padding lane, which touches no state
    got0 = torch.cat([a[:5], b, c[1:]])
    scale = want[0].abs().max()
    assert (got0.double() - want[0]).abs().max() <= 2e-5 * scale
    assert (a[5:].double() - want[1]).abs().max() <= 2e-5 * want[1].abs().max()
    assert torch.equal(c[:1], torch.zeros_like(c[:1]))
    state[2].zero_()                               # the slot is used again
    d = run([(2, hs[2])])
    assert (d.double() - want[2]).abs().max() <= 2e-5 * want[2].abs().max()
    assert torch.isnan(state[1]).all()             # the slot nobody had stays untouched


def latent_setup(H, rank, rot, page_size, num_pages, dtype):
    pages = torch.full((num_pages, 1, 1, page_size, rank + rot), float("nan"), device=DEV, dtype=dtype)
    return pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot,page_size,far", [(40, 8, 16, 15), (64, 16, 16, 16), (22, 6, 8, 3), (128, 32, 32, 31),
                                                    (24, 4, 16, 0)])
def test_latent_attention_finds_one_far_key(dtype, rank, rot, page_size, far):
    """700 cached rows in shuffled pages of a pool that is otherwise NaN; the query of every head
    points at ONE row far back (at, or next to, a page's border): the output is that row."""
    from torchlet_b200 import ops

    H, n = 3, 700
    dk = rank + rot
    num_pages = -(-n // page_size) + 5
    pages = latent_setup(H, rank, rot, page_size, num_pages, dtype)
    order = torch.randperm(num_pages - 1, generator=torch.Generator().manual_seed(1))[: -(-n // page_size)] + 1
    rows = rand(n, dk, seed=2, scale=0.02)  # every other row scores 60 * N(0, 0.02): far below 60
    rows[far] = rand(dk, seed=3, scale=1.0)
    rows[far] /= rows[far].norm()
    flat = pages.view(num_pages * page_size, dk)
    index = order.repeat_interleave(page_size)[:n] * page_size + torch.arange(n) % page_size
    flat[index.to(DEV)] = rows.to(DEV, dtype)
    table = torch.zeros(2, len(order) + 2, dtype=torch.int32, device=DEV)
    table[1, :len(order)] = order.to(DEV, torch.int32)
    q = (rows[far].to(dtype).float() * 60.0).repeat(H, 1)  # score of the far row: 60 |row|^2, of the others about 0
    q_abs = torch.stack([q, q]).to(DEV, dtype).contiguous()  # two query tokens, the last and one in the middle
    positions = torch.tensor([n - 1, max(far, 350)], dtype=torch.int32, device=DEV)
    token_req = torch.tensor([1, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(2, H * rank, device=DEV, dtype=dtype)
    ops.latent_attention(q_abs.view(2, H * dk), pages, table, token_req, positions, out, 2, H, dk, rank, page_size, 1.0)
    want = rows[far, :rank].to(dtype).float()
    got = out.float().cpu().view(2, H, rank)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= (2e-2 if dtype == torch.bfloat16 else 1e-3)
    # and a query BEFORE the far row must not see it: its output is far from that row
    if far > 0:
        positions = torch.tensor([far - 1, far - 1], dtype=torch.int32, device=DEV)
        ops.latent_attention(q_abs.view(2, H * dk), pages, table, token_req, positions, out, 2, H, dk, rank, page_size, 1.0)
        got = out.float().cpu().view(2, H, rank)
        assert torch.isfinite(got).all() and (got - want).abs().max() > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,rot,dims,V,rank", [(3, 16, 8, 4, 24, 40), (1, 12, 6, 6, 10, 22), (4, 32, 16, 16, 32, 64)])
def test_latent_attention_kernels_against_expanded_keys_and_values(dtype, H, D, rot, dims, V, rank):
    """prepare, absorb_q, attention and expand_o together against attention over expanded keys and
    values: the latent-space form must give what the per-head keys and values give."""
    from torchlet_b200 import ops

    T, page_size, eps, base, scale, q_rank = 45, 8, 1e-5, 700.0, 0.3, 16
    mixer = {"heads": H, "dim": D, "rot_dim": rot, "vdim": V, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
             "rot": {"base": base, "dims": dims}}
    shapes = {"dq": (q_rank, 56), "dq.norm": (q_rank,), "uq": (H * (D + rot), q_rank), "dkv": (rank + rot, 56),
              "dkv.norm": (rank,), "uk": (H * D, rank), "uv": (H * V, rank), "o": (56, H * V)}
    w = {}
    for i, (name, shape) in enumerate(shapes.items()):
        t = rand(*shape, seed=50 + i, scale=1.0 if len(shape) == 1 else 2.0 / math.sqrt(shape[-1]))
        w["m." + name] = (1 + 0.1 * t if name.endswith("norm") else t).bfloat16().float()
    h = rand(T, 56, seed=70)
    wd = {k: v.double() for k, v in w.items()}
    positions = torch.arange(T)
    kv = plain.latent_kv(h.double(), wd, "m.", mixer, eps, positions)
    want = plain.latent_attention(h.double(), wd, "m.", mixer, eps, positions, kv)

    dev = lambda name, dt=dtype: w["m." + name].to(DEV, dt).contiguous()
    down = (h.to(DEV) @ torch.cat([w["m.dq"], w["m.dkv"]]).to(DEV).T).contiguous()
    num_pages = -(-T // page_size) + 2
    pages = torch.full((num_pages, 1, 1, page_size, rank + rot), float("nan"), device=DEV, dtype=dtype)
    table = torch.arange(num_pages - 1, 0, -1, dtype=torch.int32, device=DEV).view(1, -1).contiguous()  # pages in reverse
    pos = positions.to(DEV, torch.int32)
    req = torch.zeros(T, dtype=torch.int32, device=DEV)
    i = torch.arange(dims // 2, dtype=torch.float64)
    inv_freq = (base ** (-2.0 * i / dims)).float().to(DEV)
    c_q = torch.empty(T, q_rank, device=DEV, dtype=dtype)
    ops.latent_prepare(down, q_rank, rank, rot, dims, dev("dq.norm", torch.float32), dev("dkv.norm", torch.float32),
                       inv_freq, eps, pos, req, table, pages, page_size, c_q, write_kv=True)
    q = (c_q.float() @ dev("uq", torch.float32).T).contiguous()
    q_abs = torch.empty(T, H * (rank + rot), device=DEV, dtype=dtype)
    ops.latent_absorb_q(q, dev("uk"), inv_freq, pos, q_abs, H, D, rot, dims, rank)
    o_lat = torch.empty(T, H * rank, device=DEV, dtype=dtype)
    ops.latent_attention(q_abs, pages, table, req, pos, o_lat, T, H, rank + rot, rank, page_size, scale)
    out = torch.empty(T, H * V, device=DEV, dtype=dtype)
    ops.latent_expand_o(o_lat, dev("uv"), out, H, V, rank)
    got = (out.float() @ dev("o", torch.float32).T).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (got - want).abs().max() <= tol * want.abs().max()
    # the cache rows themselves: latent and rotated key part
    flat = pages.view(num_pages * page_size, rank + rot).float().cpu()
    where = (table[0].cpu().long()[positions // page_size]) * page_size + positions % page_size
    cached = flat[where].double()
    row_tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (cached[:, :rank] - kv[0]).abs().max() <= row_tol * kv[0].abs().max()
    assert (cached[:, rank:] - kv[1]).abs().max() <= row_tol * kv[1].abs().max()


@pytest.mark.parametrize("H,rank,rot", [(3, 48, 16), (16, 128, 16), (5, 144, 32), (8, 256, 32), (70, 64, 16), (4, 512, 64)])
def test_tensor_core_latent_attention_equals_the_plain_kernel(H, rank, rot):
    """The mma.sync kernel against the one-warp-a-row kernel on the same cache: prompt portions with
    a cached prefix, single tokens with their keys split over several CTAs, requests of unequal
    length in one step; pages shuffled, the rest of the pool NaN."""
    from torchlet_b200 import ops

    dk, page_size = rank + rot, 16
    assert ops.latent_attention_mma_supported(dk, rank)
    lens = [(130, 37), (0, 5), (700, 1), (63, 66)]  # (cached before, new tokens)
    total = sum(b + q for b, q in lens)
    num_pages = sum(-(-(b + q) // page_size) for b, q in lens) + 3
    pages = torch.full((num_pages, 1, 1, page_size, dk), float("nan"), device=DEV, dtype=torch.bfloat16)
    order = (torch.randperm(num_pages - 1, generator=torch.Generator().manual_seed(5)) + 1).tolist()
    width = max(-(-(b + q) // page_size) for b, q in lens)
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    flat = pages.view(num_pages * page_size, dk)
    for r, (b, q) in enumerate(lens):
        n = -(-(b + q) // page_size)
        mine = [order.pop() for _ in range(n)]
        table[r, :n] = torch.tensor(mine)
        rows = rand(b + q, dk, seed=60 + r, scale=0.5).bfloat16()
        index = torch.tensor(mine).repeat_interleave(page_size)[:b + q] * page_size + torch.arange(b + q) % page_size
        flat[index.to(DEV)] = rows.to(DEV)
    T = sum(q for _, q in lens)
    q_abs = rand(T, H * dk, seed=70, scale=0.6).bfloat16().to(DEV)
    indptr = torch.tensor([0] + torch.tensor([q for _, q in lens]).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    before = torch.tensor([b for b, _ in lens], dtype=torch.int32, device=DEV)
    token_req = torch.cat([torch.full((q,), r, dtype=torch.int32) for r, (_, q) in enumerate(lens)]).to(DEV)
    positions = torch.cat([torch.arange(b, b + q, dtype=torch.int32) for b, q in lens]).to(DEV)
    table = table.to(DEV)
    want = torch.empty(T, H * rank, device=DEV, dtype=torch.bfloat16)
    ops.latent_attention(q_abs, pages, table, token_req, positions, want, T, H, dk, rank, page_size, 0.2)
    tile_req, tile_row = [], []
    for r, (_, q) in enumerate(lens):
        for row in range(0, q * H, 64):
            tile_req.append(r)
            tile_row.append(row)
    got = torch.full_like(want, float("nan"))
    ops.latent_attention_mma(q_abs, pages, table, indptr, before, torch.tensor(tile_req, dtype=torch.int32, device=DEV),
                             torch.tensor(tile_row, dtype=torch.int32, device=DEV), len(tile_req), got, T, H, dk, rank,
                             page_size, 0.2)
    assert torch.isfinite(got.float()).all()
    assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()
    # single tokens, keys split over CTAs (more splits than some requests have key tiles)
    singles = [(700, 1), (5, 1), (64, 1), (255, 1)]
    sel = [0, 1, 3]  # requests of the cache above that are long enough: 167, 5 and 129 tokens hold
    lens1 = [(lens[0][0] + lens[0][1] - 1, 1), (lens[1][0] + lens[1][1] - 1, 1), (lens[3][0] + lens[3][1] - 1, 1), (700, 1)]
    reqs = [0, 1, 3, 2]
    T1 = len(reqs)
    q1 = rand(T1, H * dk, seed=71, scale=0.6).bfloat16().to(DEV)
    table1 = table[torch.tensor(reqs, device=DEV)].contiguous()
    indptr1 = torch.arange(T1 + 1, dtype=torch.int32, device=DEV)
    before1 = torch.tensor([b for b, _ in lens1], dtype=torch.int32, device=DEV)
    req1 = torch.arange(T1, dtype=torch.int32, device=DEV)
    want1 = torch.empty(T1, H * rank, device=DEV, dtype=torch.bfloat16)
    ops.latent_attention(q1, pages, table1, req1, before1, want1, T1, H, dk, rank, page_size, 0.2)
    for splits in (1, 3, 16):
        got1 = torch.full_like(want1, float("nan"))
        ops.latent_attention_mma(q1, pages, table1, indptr1, before1, None, None, T1 * (-(-H // 64)), got1, T1, H, dk,
                                 rank, page_size, 0.2, splits)
        assert torch.isfinite(got1.float()).all(), splits
        assert (got1.float() - want1.float()).abs().max() <= 2e-2 * want1.float().abs().max(), splits


@pytest.mark.parametrize("tokens", [1, 8, 70, 300])
def test_clamped_glu_in_the_epilogue_of_the_product(tokens):
    """gate and up as one tensor-core product whose epilogue clamps and gates, against the plain
    formula on the same bfloat16 operands; many values lie beyond the limit on either side."""
    from torchlet_b200 import ops
    from torchlet_b200.parts import swiglu_bf16

    hidden, inter, limit = 64, 48, 0.9
    x = rand(tokens, hidden, seed=90).bfloat16()
    gate, up = rand(inter, hidden, seed=91, scale=0.3).bfloat16(), rand(inter, hidden, seed=92, scale=0.3).bfloat16()
    g = torch.clamp(x.double() @ gate.double().T, max=limit)
    u = torch.clamp(x.double() @ up.double().T, min=-limit, max=limit)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    assert (x.double() @ gate.double().T > limit).any() and (x.double() @ up.double().T < -limit).any()
    out = torch.empty(tokens, inter, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc_glu(x.to(DEV), swiglu_bf16.interleave(gate.to(DEV), up.to(DEV)), out, limit, 1.702)
    assert (out.cpu().double() - want).abs().max() <= 1e-2 * want.abs().max()

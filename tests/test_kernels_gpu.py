"""Each kernel alone against a plain float32 formula in torch, at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ACT = [torch.float32, torch.bfloat16]


def ops():
    from safetyraise_lmengine_b200.kernels import ops as o
    return o


def tol(dt):
    return dict(rtol=1e-5, atol=1e-5) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("H", [1, 5, 255, 256, 257, 4096])
@pytest.mark.parametrize("wdt", ACT)
def test_embed_gather(H, wdt):
    g = torch.Generator(device=DEV).manual_seed(1)
    table = torch.randn(37, H, device=DEV, generator=g).to(wdt)
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, H, device=DEV)
    bad = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embed_gather(ids, table, out, bad)
    assert torch.equal(out, table.float()[ids.long()]) and bad.item() == 0
    ids[2] = 37
    ops().embed_gather(ids, table, out, bad)
    assert bad.item() == 1 and torch.all(out[2] == 0)


@pytest.mark.parametrize("H", [4, 5, 255, 256, 257, 1000, 4096, 5120])
@pytest.mark.parametrize("dt", ACT)
@pytest.mark.parametrize("eps", [1e-6, 1e-2])
def test_add_rmsnorm(H, dt, eps):
    g = torch.Generator(device=DEV).manual_seed(2)
    T = 7
    res = torch.randn(T, H, device=DEV, generator=g) * 3
    delta = torch.randn(T, H, device=DEV, generator=g).to(dt)
    w = 1 + 0.1 * torch.randn(H, device=DEV, generator=g)
    x = res + delta.float()
    ref = x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float() * w
    out = torch.empty(T, H, device=DEV, dtype=dt)
    r = res.clone()
    ops().add_rmsnorm(r, delta, w, eps, out)
    assert torch.allclose(r, x, rtol=0, atol=0)
    assert torch.allclose(out.float(), ref, **tol(dt))
    # gathered rows, residual untouched, no delta
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, H, device=DEV, dtype=dt)
    r2 = res.clone()
    ops().add_rmsnorm(r2, None, w, eps, out2, rows=rows)
    ref2 = res * torch.rsqrt((res.double() ** 2).mean(-1, keepdim=True) + eps).float() * w
    assert torch.equal(r2, res)
    assert torch.allclose(out2.float(), ref2[rows.long()], **tol(dt))
    # gathered rows with delta: residual untouched
    ops().add_rmsnorm(r2, delta, w, eps, out2, rows=rows)
    assert torch.equal(r2, res) and torch.allclose(out2.float(), ref[rows.long()], **tol(dt))


@pytest.mark.parametrize("I", [1, 5, 257, 12288])
@pytest.mark.parametrize("dt", ACT)
def test_swiglu(I, dt):
    g = torch.Generator(device=DEV).manual_seed(3)
    gu = (torch.randn(9, 2 * I, device=DEV, generator=g) * 4).to(dt)
    out = torch.empty(9, I, device=DEV, dtype=dt)
    ops().swiglu(gu, out)
    gate, up = gu.float()[:, :I], gu.float()[:, I:]
    ref = gate * torch.sigmoid(gate) * up
    assert torch.allclose(out.float(), ref, **tol(dt))


@pytest.mark.parametrize("theta, rd", [(1e4, 16), (1e6, 128), (5e5, 48)])
def test_rope_table(theta, rd):
    pos = torch.tensor([0, 1, 2, 77, 4095, 131071], dtype=torch.int32, device=DEV)
    half = rd // 2
    cos = torch.empty(len(pos), half, device=DEV)
    sin = torch.empty_like(cos)
    ops().rope_table(pos, cos, sin, theta, rd)
    i = torch.arange(half, dtype=torch.float64)
    ang = pos.cpu().double()[:, None] / (theta ** (2 * i / rd))[None, :]
    assert torch.allclose(cos.cpu().double(), torch.cos(ang), rtol=0, atol=1e-7)
    assert torch.allclose(sin.cpu().double(), torch.sin(ang), rtol=0, atol=1e-7)


def ref_norm_rope(x, w, eps, cos, sin, half):
    # x [T, heads, hd] float32
    if w is not None:
        x = x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float() * w
    l, r = x[..., :half], x[..., half:2 * half]
    c, s = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    out[..., :half] = l * c - r * s
    out[..., half:2 * half] = r * c + l * s
    return out


@pytest.mark.parametrize("nq, nkv, hd, rd", [(4, 2, 16, 16), (5, 1, 48, 48), (8, 8, 128, 128), (3, 3, 80, 40),
                                             (6, 2, 256, 256)])
@pytest.mark.parametrize("dt", ACT)
@pytest.mark.parametrize("with_norm", [True, False])
def test_qk_norm_rope_append(nq, nkv, hd, rd, dt, with_norm):
    g = torch.Generator(device=DEV).manual_seed(4)
    T, pages, ps = 11, 9, 4
    eps = 1e-5
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=DEV, generator=g).to(dt)
    qw = (1 + 0.1 * torch.randn(hd, device=DEV, generator=g)) if with_norm else None
    kw = (1 + 0.1 * torch.randn(hd, device=DEV, generator=g)) if with_norm else None
    pos = torch.tensor([3, 4, 5, 0, 1, 2, 3, 100, 101, 7, 8], dtype=torch.int32, device=DEV)
    half = rd // 2
    cos = torch.empty(T, half, device=DEV)
    sin = torch.empty_like(cos)
    ops().rope_table(pos, cos, sin, 1e4, rd)
    slots = torch.randperm(pages * ps, device=DEV, generator=g)[:T].to(torch.int32)
    slots[5] = -1                                   # this token's keys are not kept
    kc = torch.full((pages, nkv, ps, hd), 7.0, device=DEV, dtype=dt)     # [page, kv head, token, dim]
    vc = torch.full((pages, nkv, ps, hd), 7.0, device=DEV, dtype=dt)
    q = torch.empty(T, nq * hd, device=DEV, dtype=dt)
    ops().qk_norm_rope_append(qkv, q, kc, vc, qw, kw, eps, cos, sin, slots, nq, nkv, hd, half)
    x = qkv.float().view(T, nq + 2 * nkv, hd)
    q_ref = ref_norm_rope(x[:, :nq], qw, eps, cos, sin, half)
    k_ref = ref_norm_rope(x[:, nq:nq + nkv], kw, eps, cos, sin, half)
    v_ref = x[:, nq + nkv:]
    assert torch.allclose(q.float().view(T, nq, hd), q_ref, **tol(dt))
    kflat = kc.float().permute(0, 2, 1, 3).reshape(pages * ps, nkv, hd)
    vflat = vc.float().permute(0, 2, 1, 3).reshape(pages * ps, nkv, hd)
    for t in range(T):
        if slots[t] < 0:
            continue
        assert torch.allclose(kflat[slots[t]], k_ref[t], **tol(dt))
        assert torch.equal(vflat[slots[t]], v_ref[t].to(dt).float())
    untouched = torch.ones(pages * ps, dtype=torch.bool, device=DEV)
    untouched[slots[slots >= 0].long()] = False
    assert torch.all(kflat[untouched] == 7.0) and torch.all(vflat[untouched] == 7.0)
    # a step that only reads another step's cache leaves it alone
    kc2, vc2 = kc.clone(), vc.clone()
    ops().qk_norm_rope_append(qkv, q, kc2, vc2, qw, kw, eps, cos, sin, slots, nq, nkv, hd, half, write_kv=False)
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)


def ref_paged_attention(q, kc, vc, tables, entry_of_token, positions, nq, nkv, hd, ps, scale, window):
    T = q.shape[0]
    out = torch.zeros(T, nq, hd, dtype=torch.float64)
    qd, kd, vd = q.double().cpu().view(T, nq, hd), kc.double().cpu(), vc.double().cpu()
    for t in range(T):
        e, p = int(entry_of_token[t]), int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        js = torch.arange(lo, p + 1)
        rows = torch.tensor([tables[e][j // ps] for j in js.tolist()]) * ps + js % ps
        kf = kd.permute(0, 2, 1, 3).reshape(-1, nkv, hd)[rows]      # caches are [page, kv head, token, dim]
        vf = vd.permute(0, 2, 1, 3).reshape(-1, nkv, hd)[rows]
        for h in range(nq):
            kh = h // (nq // nkv)
            s = (kf[:, kh] @ qd[t, h]) * scale
            pr = torch.softmax(s, 0)
            out[t, h] = pr @ vf[:, kh]
    return out


def make_paged_case(nq, nkv, hd, ps, dt, lens_q, lens_kv, seed=5, pages=64):
    g = torch.Generator(device=DEV).manual_seed(seed)
    n = len(lens_q)
    T = sum(lens_q)
    kc = torch.randn(pages, nkv, ps, hd, device=DEV, generator=g).to(dt)
    vc = torch.randn(pages, nkv, ps, hd, device=DEV, generator=g).to(dt)
    q = torch.randn(T, nq * hd, device=DEV, generator=g).to(dt)
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    tables, used = [], 0
    for kv in lens_kv:
        need = (kv + ps - 1) // ps
        tables.append(perm[used:used + need])
        used += need
    assert used <= pages
    width = max(len(t) for t in tables)
    bt = torch.zeros(n, width, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    eot, pos = [], []
    for i, (ql, kv) in enumerate(zip(lens_q, lens_kv)):
        eot += [i] * ql
        pos += list(range(kv - ql, kv))
    return q, kc, vc, tables, bt.to(DEV), torch.tensor(eot, dtype=torch.int32, device=DEV), \
        torch.tensor(pos, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("nq, nkv, hd, ps", [(4, 2, 16, 4), (6, 1, 32, 16), (8, 2, 128, 16), (5, 5, 80, 8),
                                             (2, 1, 256, 32)])
@pytest.mark.parametrize("dt", ACT)
@pytest.mark.parametrize("window", [0, 9])
def test_paged_attention_simt(nq, nkv, hd, ps, dt, window):
    lens_q, lens_kv = [1, 7, 33, 1, 2], [1, 40, 33, 65, 100]
    q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, dt, lens_q, lens_kv)
    out = torch.empty_like(q)
    scale = 1 / math.sqrt(hd)
    ops().paged_attention_simt(q, kc, vc, out, bt, eot, pos, nq, nkv, hd, ps, scale, window)
    ref = ref_paged_attention(q, kc, vc, tables, eot.cpu(), pos.cpu(), nq, nkv, hd, ps, scale, window)
    t = dict(rtol=1e-4, atol=1e-5) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    assert torch.allclose(out.float().cpu().view(-1, nq, hd).double(), ref, **t)


def test_paged_attention_finds_one_far_key():
    """One key among hundreds carries the mass: a kernel that skips or misplaces it shows at once."""
    nq, nkv, hd, ps = 4, 2, 32, 16
    q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.float32, [1], [700], pages=48)
    out = torch.empty_like(q)
    for far in (0, 15, 16, 333, 699):
        kc2 = kc * 0.01
        page, off = tables[0][far // ps], far % ps
        kc2[page, :, off] = q.view(nq, hd)[0::2] * 4.0     # heads 0 and 2 -> kv heads 0 and 1
        ops().paged_attention_simt(q, kc2, vc, out, bt, eot, pos, nq, nkv, hd, ps, 1.0, 0)
        got = out.view(nq, hd)
        for h, kh in ((0, 0), (2, 1)):
            assert torch.allclose(got[h], vc[page, kh, off], atol=1e-3), (far, h)


@pytest.mark.parametrize("M, N, K", [(1, 1, 1), (3, 5, 7), (64, 64, 16), (65, 129, 33), (17, 384, 96),
                                     (200, 255, 257), (8, 4096, 1024)])
@pytest.mark.parametrize("dts", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                 (torch.bfloat16, torch.float32)])
def test_gemm_tn_simt(M, N, K, dts):
    adt, odt = dts
    g = torch.Generator(device=DEV).manual_seed(6)
    a = torch.randn(M, K, device=DEV, generator=g).to(adt)
    w = torch.randn(N, K, device=DEV, generator=g).to(adt)
    out = torch.empty(M, N, device=DEV, dtype=odt)
    ops().gemm_tn_simt(a, w, out)
    ref = (a.double() @ w.double().T)
    if odt == torch.float32:
        assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-4 * math.sqrt(K))
    else:
        assert torch.allclose(out.double(), ref, rtol=1e-2, atol=1e-2 * math.sqrt(K))


def test_gemm_rows_do_not_depend_on_the_batch():
    g = torch.Generator(device=DEV).manual_seed(8)
    a = torch.randn(130, 300, device=DEV, generator=g)
    w = torch.randn(77, 300, device=DEV, generator=g)
    full = torch.empty(130, 77, device=DEV)
    ops().gemm_tn_simt(a, w, full)
    one = torch.empty(1, 77, device=DEV)
    ops().gemm_tn_simt(a[97:98].contiguous(), w, one)
    assert torch.equal(one[0], full[97])


def test_argmax_ties_go_to_the_lowest_id():
    logits = torch.zeros(4, 1000, device=DEV)
    logits[0, [5, 700]] = 3.0
    logits[1, 999] = 1.0
    logits[2] = -1.0
    logits[3, 512] = 2.0
    logits[3, 513] = 2.0
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    bad = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().argmax(logits, out, bad)
    assert out.tolist() == [5, 999, 0, 512] and bad.item() == 0
    big = torch.randn(3, 151936, device=DEV)
    out3 = torch.empty(3, dtype=torch.int32, device=DEV)
    ops().argmax(big, out3, bad)
    assert out3.tolist() == big.argmax(-1).tolist()
    big[1, 7] = float("nan")
    ops().argmax(big, out3, bad)
    assert bad.item() == 1


@pytest.mark.parametrize("M, N, K, splits", [
    (1, 128, 64, 1), (8, 384, 96, 1), (16, 192, 64, 1), (17, 200, 72, 1), (33, 4096, 4096, 4),
    (64, 2560, 4096, 1), (64, 512, 1024, 3), (100, 384, 256, 1), (129, 640, 512, 2), (300, 640, 520, 1),
    (2048, 1024, 512, 1), (5, 6144, 4096, None), (8, 4096, 12288, None), (257, 128, 8, 1),
    (40, 7168, 5120, None), (200, 5120, 17408, 1), (64, 10240, 5120, None), (520, 1280, 25600, 1),
    # splits of 2 to 8 add their sums inside a thread-block cluster, more through the workspace
    (129, 640, 2048, 4), (260, 1000, 1536, 3), (50, 264, 4096, 8), (20, 136, 8192, 12), (64, 4096, 4096, 6),
    (128, 4096, 12288, None), (256, 6144, 4096, None), (7, 392, 1024, 5)])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32])
def test_gemm_tn_tcgen05(M, N, K, splits, odt):
    g = torch.Generator(device=DEV).manual_seed(M * 7 + N)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=odt)
    ops().gemm_tn_tcgen05(a, w, out, splits=splits)
    assert ops().gemm_error_flag(a.device) == 0
    ref = a.double() @ w.double().T
    if odt == torch.float32:
        assert torch.allclose(out.double(), ref, rtol=1e-4, atol=2e-4 * math.sqrt(K))
        twin = torch.empty(M, N, device=DEV)
        ops().gemm_tn_simt(a, w, twin)
        assert torch.allclose(out, twin, rtol=1e-4, atol=2e-4 * math.sqrt(K))
    else:
        assert torch.allclose(out.double(), ref, rtol=1e-2, atol=1e-2 * math.sqrt(K))
    # twice in a row: the split-K counters were left clean
    out2 = torch.empty_like(out)
    ops().gemm_tn_tcgen05(a, w, out2, splits=splits)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("M, N, K, dealt", [
    # token tiles of 128 whose tiles do not fill the last round: the persistent kernel deals the k-blocks of
    # the left-over tiles out evenly, parts of a tile meet in the workspace and are added in a fixed order
    (128, 22000, 4096, True), (128, 24576, 2048, True), (100, 24000, 2304, True),
    # a few hundred tokens and a narrow output: two rounds of 128 x 128 tiles, or one of pairs' tiles (chosen);
    # tiles for at most 70 % of the pairs and a long K: their k-blocks are dealt out evenly to all pairs
    (512, 6000, 2048, False), (500, 5120, 6400, False), (512, 4096, 1024, False), (512, 5000, 14400, True),
    (400, 6100, 12296, True), (260, 6300, 16008, True),
    # token tiles of 256: a pair of SMs (cta_group::2) per tile of 256 weight rows x 256 tokens; ragged
    # token counts, a last tile whose second half lies beyond the weight rows, K no multiple of 64
    (2048, 6144, 4096, False), (900, 6144, 2048, False), (1100, 24576, 1792, False), (1300, 4224, 3000, False),
    (2050, 5008, 520, False), (257, 19072, 72, False), (512, 6144, 4096, False), (640, 4096, 6400, False)])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_persistent_forms(M, N, K, dealt, odt):
    assert (ops().gemm_dealt_tiles(M, N, K) > 0) == dealt
    g = torch.Generator(device=DEV).manual_seed(M + N)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=odt)
    ops().gemm_tn_tcgen05(a, w, out)
    assert ops().gemm_error_flag(a.device) == 0
    ref = a.float() @ w.float().T
    if odt == torch.float32:
        assert torch.allclose(out, ref, rtol=1e-4, atol=2e-4 * math.sqrt(K))
    else:
        assert torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-2 * math.sqrt(K))
    for _ in range(3):                 # the same bits on every run, and the counters were left clean
        out2 = torch.full_like(out, float("nan"))
        ops().gemm_tn_tcgen05(a, w, out2)
        assert torch.equal(out, out2)
    # with the SwiGLU epilogue
    if N % 16 == 0:
        out3 = torch.full((M, N // 2), float("nan"), device=DEV, dtype=odt)
        ws = (w.float() / math.sqrt(K) * 2).to(torch.bfloat16)
        ops().gemm_tn_tcgen05(a, ws, out3, swiglu8=True)
        full = (a.float() @ ws.float().T).view(M, N // 16, 2, 8)
        ref3 = (torch.nn.functional.silu(full[:, :, 0]) * full[:, :, 1]).reshape(M, N // 2)
        assert torch.allclose(out3.float(), ref3, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nq, nkv, hd, rd", [(4, 2, 16, 16), (3, 1, 48, 20), (2, 2, 128, 128), (6, 2, 64, 32)])
@pytest.mark.parametrize("dt", ACT)
def test_qk_norm_rope_append_interleaved_pairs(nq, nkv, hd, rd, dt):
    """Pairs (2i, 2i+1) of the first rd elements of a head, as other rotary encodings use them."""
    g = torch.Generator(device=DEV).manual_seed(6)
    T, pages, ps, eps = 9, 6, 4, 1e-6
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=DEV, generator=g).to(dt)
    qw = 1 + 0.1 * torch.randn(hd, device=DEV, generator=g)
    kw = 1 + 0.1 * torch.randn(hd, device=DEV, generator=g)
    pos = torch.tensor([0, 1, 2, 50, 51, 7, 8, 9, 300], dtype=torch.int32, device=DEV)
    half = rd // 2
    cos, sin = torch.empty(T, half, device=DEV), torch.empty(T, half, device=DEV)
    ops().rope_table(pos, cos, sin, 1e4, rd)
    slots = torch.randperm(pages * ps, device=DEV, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=dt)
    vc = torch.zeros_like(kc)
    q = torch.empty(T, nq * hd, device=DEV, dtype=dt)
    ops().qk_norm_rope_append(qkv, q, kc, vc, qw, kw, eps, cos, sin, slots, nq, nkv, hd, half, interleaved=True)

    def ref(x, w):
        x = x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float() * w
        out = x.clone()
        e, o = x[..., 0:rd:2], x[..., 1:rd:2]
        c, sn = cos[:, None, :], sin[:, None, :]
        out[..., 0:rd:2] = e * c - o * sn
        out[..., 1:rd:2] = o * c + e * sn
        return out

    x = qkv.float().view(T, nq + 2 * nkv, hd)
    assert torch.allclose(q.float().view(T, nq, hd), ref(x[:, :nq], qw), **tol(dt))
    kflat = kc.float().permute(0, 2, 1, 3).reshape(pages * ps, nkv, hd)
    assert torch.allclose(kflat[slots.long()], ref(x[:, nq:nq + nkv], kw), **tol(dt))
    if rd == hd and hd >= 16:       # and it is not the half-split rotation
        assert not torch.allclose(q.float().view(T, nq, hd), ref_norm_rope(x[:, :nq], qw, eps, cos, sin, half), **tol(dt))


def test_gemm_tcgen05_tensor_maps_survive_the_emptying_of_their_cache():
    """The cache of tensor maps is emptied when it is full.  A product looks up the weight's map, then
    the activations' map: when the second lookup empties the cache, the first map must still be whole
    (it is copied out under the lock, never pointed to)."""
    import ctypes as C
    lib = ops().lib
    limit = C.c_int(0)
    lib.srlm_gemm_tcgen05_map_cache(C.byref(limit))
    g = torch.Generator(device=DEV).manual_seed(8)
    N, K = 128, 64
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    big = (torch.randn(limit.value + 40, K, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    out = torch.empty(9, N, device=DEV, dtype=torch.float32)
    emptied = 0
    for i in range(limit.value + 30):                                # every start row is a new key for the activations
        before = lib.srlm_gemm_tcgen05_map_cache(None)
        ops().gemm_tn_tcgen05(big[i:i + 9], w, out)
        if lib.srlm_gemm_tcgen05_map_cache(None) < before:           # this call emptied the cache between its lookups
            emptied += 1
            assert torch.allclose(out, big[i:i + 9].float() @ w.float().t(), rtol=1e-3, atol=1e-3), i
    assert emptied >= 1
    assert ops().gemm_error_flag(torch.device(DEV)) == 0


def test_host_plans_agree_with_the_kernels_and_the_device():
    """The host-side plans repeat two facts of the device side: the SM count they are tuned for, and the
    rule by which the tensor-core product picks its token tile."""
    import ctypes as C
    from safetyraise_lmengine_b200.kernels.library import KernelLibrary
    assert ops().sm_count(torch.device(DEV)) == KernelLibrary.SMS
    least = C.c_int(0)
    for M in (1, 16, 17, 33, 64, 65, 128, 129, 256, 300, 512, 2048, 5000):
        for N in (128, 4096, 5120, 6144, 12200, 24576, 151936):
            assert ops().lib.srlm_gemm_tcgen05_token_tile(M, N, C.byref(least)) == KernelLibrary.gemm_token_tile(M, N), (M, N)
    assert least.value == KernelLibrary.BN256_MIN_TILES


def test_gemm_tcgen05_finds_each_k_and_row():
    """Identity-like operands: a misplaced row, column or k block shows as a wrong integer."""
    K, N, M = 256, 256, 40
    w = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
    w[torch.arange(N), torch.arange(N) % K] = 1.0
    a = (torch.arange(M * K, device=DEV).reshape(M, K) % 251).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.float32)
    ops().gemm_tn_tcgen05(a, w, out, splits=1)
    assert torch.equal(out, a.float()[:, torch.arange(N, device=DEV) % K])


def test_gemm_tcgen05_refuses_what_tma_cannot_address():
    from safetyraise_lmengine_b200.errors import ShapeError
    a = torch.zeros(4, 100, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(8, 100, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(4, 8, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ShapeError):
        ops().gemm_tn_tcgen05(a, w, out)
    ops().gemm(a, w, out)              # the dispatcher falls back to the FMA kernel for such a width


ATT_CASES = [(4, 2, 16, 4), (6, 1, 32, 16), (32, 8, 128, 16), (5, 5, 80, 8), (2, 1, 256, 32), (8, 2, 64, 16),
             (12, 4, 112, 16)]


@pytest.mark.parametrize("nq, nkv, hd, ps", ATT_CASES)
@pytest.mark.parametrize("window", [0, 37])
def test_paged_attention_rows_mma(nq, nkv, hd, ps, window):
    lens_q, lens_kv = [1, 7, 33, 1, 2, 150], [1, 40, 33, 65, 100, 300]
    q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.bfloat16, lens_q, lens_kv, pages=160)
    g = nq // nkv
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lens_kv, dtype=torch.int32, device=DEV)
    work = torch.tensor([(e, t) for e, ql in enumerate(lens_q) for t in range((ql * g + 63) // 64)],
                        dtype=torch.int32, device=DEV)
    out = torch.full_like(q, float("nan"))
    scale = 1 / math.sqrt(hd)
    ops().paged_attention_rows(q, kc, vc, out, bt, cu, kvl, work, nq, nkv, hd, ps, scale, window)
    ref = ref_paged_attention(q, kc, vc, tables, eot.cpu(), pos.cpu(), nq, nkv, hd, ps, scale, window)
    assert torch.allclose(out.float().cpu().view(-1, nq, hd).double(), ref, rtol=2e-2, atol=2e-2)
    twin = torch.empty_like(q)
    ops().paged_attention_simt(q, kc, vc, twin, bt, eot, pos, nq, nkv, hd, ps, scale, window)
    assert torch.allclose(out.float(), twin.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nq, nkv, hd, ps", ATT_CASES)
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("nsplit", [1, 3])
def test_paged_attention_keys_mma(nq, nkv, hd, ps, window, nsplit):
    g = nq // nkv
    ql = max(1, min(3, 16 // g))
    lens_q, lens_kv = [1, ql, 1, 1, ql], [1, 40, 65, 300, 129]
    q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.bfloat16, lens_q, lens_kv, pages=160)
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lens_kv, dtype=torch.int32, device=DEV)
    n = len(lens_q)
    chunk = ((max(lens_kv) + nsplit - 1) // nsplit + 63) // 64 * 64
    part_o = torch.full((n * nkv * nsplit * 16, hd), float("nan"), device=DEV)
    part_ml = torch.full((n * nkv * nsplit * 16, 2), float("nan"), device=DEV)
    out = torch.full_like(q, float("nan"))
    scale = 1 / math.sqrt(hd)
    ops().paged_attention_keys(q, kc, vc, out, bt, cu, kvl, n, nq, nkv, hd, ps, scale, window, chunk, nsplit,
                               part_o, part_ml)
    ref = ref_paged_attention(q, kc, vc, tables, eot.cpu(), pos.cpu(), nq, nkv, hd, ps, scale, window)
    assert torch.allclose(out.float().cpu().view(-1, nq, hd).double(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("kernel", ["rows", "keys"])
def test_mma_attention_finds_one_far_key(kernel):
    nq, nkv, hd, ps = 8, 2, 64, 16
    for far in (0, 63, 64, 333, 699):
        q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.bfloat16, [1], [700], pages=48)
        kc = kc * 0.01
        page, off = tables[0][far // ps], far % ps
        kc[page, :, off] = q.view(nq, hd)[0::4] * 4.0              # heads 0 and 4 -> kv heads 0 and 1
        out = torch.empty_like(q)
        cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
        kvl = torch.tensor([700], dtype=torch.int32, device=DEV)
        if kernel == "rows":
            work = torch.tensor([[0, 0]], dtype=torch.int32, device=DEV)
            ops().paged_attention_rows(q, kc, vc, out, bt, cu, kvl, work, nq, nkv, hd, ps, 1.0, 0)
        else:
            part_o = torch.empty(2 * 4 * 16, hd, device=DEV)
            part_ml = torch.empty(2 * 4 * 16, 2, device=DEV)
            ops().paged_attention_keys(q, kc, vc, out, bt, cu, kvl, 1, nq, nkv, hd, ps, 1.0, 0, 192, 4, part_o, part_ml)
        got = out.float().view(nq, hd)
        for h, kh in ((0, 0), (4, 1)):
            assert torch.allclose(got[h], vc[page, kh, off].float(), atol=2e-2), (far, h)


@pytest.mark.parametrize("nq, nkv, hd, ps", [(32, 8, 128, 16), (8, 2, 64, 16), (4, 4, 64, 8), (16, 1, 128, 32),
                                             (6, 2, 192, 64), (2, 1, 256, 128)])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("nsplit, cluster", [(1, False), (3, False), (3, True), (5, True), (8, True)])
def test_paged_attention_decode_tma(nq, nkv, hd, ps, window, nsplit, cluster):
    """Slices of the keys merged through global partials (cluster False) or through the distributed shared
    memory of a thread-block cluster, which needs no partial buffers."""
    g = nq // nkv
    ql = max(1, min(3, 16 // g))
    lens_q, lens_kv = [1, ql, 1, 1, ql], [1, 40, 65, 300, 129]
    q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.bfloat16, lens_q, lens_kv, pages=160)
    used = torch.zeros(160, dtype=torch.bool)
    for t in tables:
        used[t] = True
    kc[~used.to(DEV)] = float("nan")                  # pages of nobody: reading them must not matter
    vc[~used.to(DEV)] = float("nan")
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lens_kv, dtype=torch.int32, device=DEV)
    n = len(lens_q)
    chunk = ((max(lens_kv) + nsplit - 1) // nsplit + 63) // 64 * 64
    part_o = part_ml = None
    if not cluster:
        part_o = torch.full((n * nkv * nsplit * 16, hd), float("nan"), device=DEV)
        part_ml = torch.full((n * nkv * nsplit * 16, 2), float("nan"), device=DEV)
    out = torch.full_like(q, float("nan"))
    scale = 1 / math.sqrt(hd)
    ops().paged_attention_decode_tma(q, kc, vc, out, bt, cu, kvl, n, nq, nkv, hd, ps, scale, window, chunk, nsplit,
                                     part_o, part_ml, cluster=cluster)
    assert ops().gemm_error_flag(q.device) == 0
    kc[~used.to(DEV)] = 0
    vc[~used.to(DEV)] = 0
    ref = ref_paged_attention(q, kc, vc, tables, eot.cpu(), pos.cpu(), nq, nkv, hd, ps, scale, window)
    assert torch.allclose(out.float().cpu().view(-1, nq, hd).double(), ref, rtol=2e-2, atol=2e-2)
    # the tail of each request's last page is poisoned too: rows nobody wrote
    for t, kv in zip(tables, lens_kv):
        if kv % ps:
            vc[t[-1], :, kv % ps:] = float("nan")
            kc[t[-1], :, kv % ps:] = float("nan")
    out2 = torch.full_like(q, float("nan"))
    ops().paged_attention_decode_tma(q, kc, vc, out2, bt, cu, kvl, n, nq, nkv, hd, ps, scale, window, chunk, nsplit,
                                     part_o, part_ml, cluster=cluster)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("nq, nkv, hd, ps", [(32, 8, 128, 16), (8, 2, 64, 16), (4, 4, 64, 8), (16, 1, 128, 32),
                                             (2, 1, 256, 128), (6, 3, 128, 64)])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("nsplit, cluster", [(1, False), (3, False), (5, True)])
@pytest.mark.parametrize("with_norm", [True, False])
def test_decode_attention_from_the_projection(nq, nkv, hd, ps, window, nsplit, cluster, with_norm):
    """Norm, rotation, append and attention in one kernel against the two kernels one after the other:
    the same cache contents and the same output, bit for bit; pages of nobody and rows nobody wrote
    hold NaN.  New positions fall on page edges, tile edges (64) and slice edges."""
    g = nq // nkv
    ql = max(1, min(3, 16 // g))
    lens_q, lens_kv = [1, ql, 1, 1, ql, 1], [1, 40, 65, 300, 129, 64]
    _, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.bfloat16, lens_q, lens_kv, pages=160)
    n, T = len(lens_q), sum(lens_q)
    gen = torch.Generator(device=DEV).manual_seed(11)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=DEV, generator=gen).to(torch.bfloat16)
    qw = (1 + 0.3 * torch.randn(hd, device=DEV, generator=gen)) if with_norm else None
    kw = (1 + 0.3 * torch.randn(hd, device=DEV, generator=gen)) if with_norm else None
    cos = torch.empty(T, hd // 2, device=DEV)
    sin = torch.empty_like(cos)
    ops().rope_table(pos, cos, sin, 10000.0, hd)
    used = torch.zeros(160, dtype=torch.bool)
    for t in tables:
        used[t] = True
    kc[~used.to(DEV)] = float("nan")
    vc[~used.to(DEV)] = float("nan")
    slot = []
    for t, ql_, kv in zip(tables, lens_q, lens_kv):
        for p_ in range(kv - ql_, kv):                    # the new positions hold NaN until the step writes them
            kc[t[p_ // ps], :, p_ % ps] = float("nan")
            vc[t[p_ // ps], :, p_ % ps] = float("nan")
            slot.append(t[p_ // ps] * ps + p_ % ps)
        if kv % ps:
            kc[t[-1], :, kv % ps:] = float("nan")
            vc[t[-1], :, kv % ps:] = float("nan")
    slot = torch.tensor(slot, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lens_kv, dtype=torch.int32, device=DEV)
    chunk = ((max(lens_kv) + nsplit - 1) // nsplit + 63) // 64 * 64
    scale = 1 / math.sqrt(hd)
    part_o = part_ml = None
    if not cluster:
        part_o = torch.full((n * nkv * nsplit * 16, hd), float("nan"), device=DEV)
        part_ml = torch.full((n * nkv * nsplit * 16, 2), float("nan"), device=DEV)
    # one after the other
    kc1, vc1 = kc.clone(), vc.clone()
    q1 = torch.empty(T, nq * hd, device=DEV, dtype=torch.bfloat16)
    out1 = torch.full_like(q1, float("nan"))
    ops().qk_norm_rope_append(qkv, q1, kc1, vc1, qw, kw, 1e-5, cos, sin, slot, nq, nkv, hd, hd // 2)
    ops().paged_attention_decode_tma(q1, kc1, vc1, out1, bt, cu, kvl, n, nq, nkv, hd, ps, scale, window, chunk,
                                     nsplit, part_o, part_ml, cluster=cluster)
    # in one kernel
    kc2, vc2 = kc.clone(), vc.clone()
    out2 = torch.full_like(q1, float("nan"))
    ops().paged_attention_decode_fused(qkv, qw, kw, 1e-5, cos, sin, True, kc2, vc2, out2, bt, cu, kvl, n, nq, nkv,
                                       hd, ps, scale, window, chunk, nsplit, part_o, part_ml, cluster=cluster)
    assert ops().gemm_error_flag(qkv.device) == 0
    assert not torch.isnan(out1).any()
    assert torch.equal(kc1.view(torch.int16), kc2.view(torch.int16))
    assert torch.equal(vc1.view(torch.int16), vc2.view(torch.int16))
    assert torch.equal(out1, out2)
    # without writing: the cache already holds the step's keys and values
    out3 = torch.full_like(q1, float("nan"))
    ops().paged_attention_decode_fused(qkv, qw, kw, 1e-5, cos, sin, False, kc1, vc1, out3, bt, cu, kvl, n, nq, nkv,
                                       hd, ps, scale, window, chunk, nsplit, part_o, part_ml, cluster=cluster)
    assert torch.equal(out1, out3)


@pytest.mark.parametrize("M, N, K", [(1, 16, 8), (1, 4096, 4096), (8, 6144, 4096), (8, 200, 72), (5, 17, 520),
                                     (9, 384, 96), (16, 4096, 12288), (13, 1000, 264), (8, 151936, 512),
                                     (8, 7168, 5120), (3, 5120, 25600)])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32])
def test_gemm_tn_skinny(M, N, K, odt):
    g = torch.Generator(device=DEV).manual_seed(M * 7 + N)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=odt)
    ops().gemm_tn_skinny(a, w, out)
    ref = a.double() @ w.double().T
    if odt == torch.float32:
        assert torch.allclose(out.double(), ref, rtol=1e-4, atol=2e-4 * math.sqrt(K))
    else:
        assert torch.allclose(out.double(), ref, rtol=1e-2, atol=1e-2 * math.sqrt(K))
    out2 = torch.empty_like(out)
    ops().gemm_tn_skinny(a, w, out2)
    assert torch.equal(out, out2)


def test_gemm_skinny_finds_each_k_and_row():
    K, N, M = 256, 256, 11
    w = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
    w[torch.arange(N), torch.arange(N) % K] = 1.0
    a = (torch.arange(M * K, device=DEV).reshape(M, K) % 251).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.float32)
    ops().gemm_tn_skinny(a, w, out)
    assert torch.equal(out, a.float()[:, torch.arange(N, device=DEV) % K])
    from safetyraise_lmengine_b200.errors import ShapeError
    with pytest.raises(ShapeError):
        ops().gemm_tn_skinny(torch.zeros(17, K, device=DEV, dtype=torch.bfloat16), w,
                             torch.empty(17, N, device=DEV, dtype=torch.float32))


@pytest.mark.parametrize("M, I, K, splits", [(1, 8, 64, 1), (8, 12288, 512, 1), (5, 24, 72, 1), (16, 256, 96, 1),
                                             (6, 2560, 264, 1),      # 320 blocks: the lean form of the weight-streaming kernel
                                             (33, 128, 256, 2), (100, 4096, 512, 1), (64, 512, 2048, 3), (300, 200, 128, 1),
                                             (100, 512, 2048, 4), (200, 136, 1024, 2), (24, 64, 8192, 10)])
def test_gemm_with_fused_swiglu(M, I, K, splits):
    """Both tensor-core products with the SwiGLU epilogue against product-then-SwiGLU."""
    g = torch.Generator(device=DEV).manual_seed(M + I)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    gate = (torch.randn(I, K, device=DEV, generator=g) / math.sqrt(K) * 2).to(torch.bfloat16)
    up = (torch.randn(I, K, device=DEV, generator=g) / math.sqrt(K) * 2).to(torch.bfloat16)
    w = torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    gd, ud = a.double() @ gate.double().T, a.double() @ up.double().T
    ref = gd * torch.sigmoid(gd) * ud
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops().gemm_tn_tcgen05(a, w, out, splits=splits, swiglu8=True)
    assert ops().gemm_error_flag(a.device) == 0
    assert torch.allclose(out.double(), ref, rtol=2e-2, atol=2e-2)
    if M <= 16:
        out2 = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
        ops().gemm_tn_skinny(a, w, out2, swiglu8=True)
        assert torch.allclose(out2.double(), ref, rtol=2e-2, atol=2e-2)
        out32 = torch.full((M, I), float("nan"), device=DEV, dtype=torch.float32)
        ops().gemm_tn_skinny(a, w, out32, swiglu8=True)
        assert torch.allclose(out32.double(), ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("nq, nkv, hd, ps", [(32, 8, 128, 16), (8, 2, 64, 16), (4, 4, 64, 8), (16, 1, 128, 32),
                                             (6, 2, 128, 64)])
@pytest.mark.parametrize("window", [0, 37])
def test_paged_attention_rows_tma(nq, nkv, hd, ps, window):
    lens_q, lens_kv = [1, 7, 33, 1, 2, 150, 300], [1, 40, 33, 65, 100, 300, 300]
    q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.bfloat16, lens_q, lens_kv, pages=260)
    used = torch.zeros(260, dtype=torch.bool)
    for t in tables:
        used[t] = True
    kc[~used.to(DEV)] = float("nan")
    vc[~used.to(DEV)] = float("nan")
    for t, kv in zip(tables, lens_kv):                 # the unwritten tail of each last page too
        if kv % ps:
            vc[t[-1], :, kv % ps:] = float("nan")
            kc[t[-1], :, kv % ps:] = float("nan")
    g = nq // nkv
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lens_kv, dtype=torch.int32, device=DEV)
    work = torch.tensor([(e, t) for e, ql in enumerate(lens_q) for t in range((ql * g + 127) // 128)],
                        dtype=torch.int32, device=DEV)
    out = torch.full_like(q, float("nan"))
    scale = 1 / math.sqrt(hd)
    ops().paged_attention_rows_tma(q, kc, vc, out, bt, cu, kvl, work, nq, nkv, hd, ps, scale, window)
    assert ops().gemm_error_flag(q.device) == 0
    kc, vc = torch.nan_to_num(kc), torch.nan_to_num(vc)
    ref = ref_paged_attention(q, kc, vc, tables, eot.cpu(), pos.cpu(), nq, nkv, hd, ps, scale, window)
    assert torch.allclose(out.float().cpu().view(-1, nq, hd).double(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nq, nkv, ps", [(32, 8, 16), (8, 2, 8), (4, 4, 32), (16, 1, 64), (6, 2, 128), (5, 5, 16)])
@pytest.mark.parametrize("window", [0, 37, 200])
@pytest.mark.parametrize("tiles", [1, 2])
def test_paged_attention_prefill_tcgen05(nq, nkv, ps, window, tiles):
    """The tcgen05 prefill attention: ragged entries, partly filled pages, pages of other requests and
    unwritten page tails poisoned with NaN, a far key that must win the softmax."""
    check_prefill_tcgen05(nq, nkv, ps, window, tiles, 1, 0)


@pytest.mark.parametrize("nq, nkv, ps", [(32, 8, 16), (4, 4, 32), (6, 2, 128)])
@pytest.mark.parametrize("window", [0, 37, 200])
@pytest.mark.parametrize("tiles, nsplit, chunk", [(2, 3, 256), (1, 2, 384), (2, 6, 128)])
def test_paged_attention_prefill_tcgen05_key_slices(nq, nkv, ps, window, tiles, nsplit, chunk):
    """The same with the keys cut into slices: slices beyond an entry's keys, slices that end inside a
    row tile's diagonal, a window that starts inside a later slice; the workspace starts as NaN."""
    check_prefill_tcgen05(nq, nkv, ps, window, tiles, nsplit, chunk)


def check_prefill_tcgen05(nq, nkv, ps, window, tiles, nsplit, chunk):
    hd = 128
    lens_q, lens_kv = [1, 7, 33, 1, 2, 150, 300, 520], [1, 40, 33, 65, 100, 300, 300, 700]
    pages = 120 + sum(-(-kv // ps) for kv in lens_kv)
    q, kc, vc, tables, bt, eot, pos = make_paged_case(nq, nkv, hd, ps, torch.bfloat16, lens_q, lens_kv, pages=pages)
    used = torch.zeros(pages, dtype=torch.bool)
    for t in tables:
        used[t] = True
    kc[~used.to(DEV)] = float("nan")
    vc[~used.to(DEV)] = float("nan")
    for t, kv in zip(tables, lens_kv):
        if kv % ps:
            vc[t[-1], :, kv % ps:] = float("nan")
            kc[t[-1], :, kv % ps:] = float("nan")
    if window == 0:
        # the last entry's last row looks hard at key 3 (a far key among hundreds)
        kc[tables[-1][3 // ps], :, 3 % ps] = 0
        kc[tables[-1][3 // ps], :, 3 % ps, 0] = 30.0
        q.view(-1, nq, hd)[-1] = 0
        q.view(-1, nq, hd)[-1, :, 0] = 30.0
    g = nq // nkv
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lens_kv, dtype=torch.int32, device=DEV)
    rows = 128 * tiles
    work = torch.tensor([(e, t) for e, ql in enumerate(lens_q) for t in reversed(range((ql * g + rows - 1) // rows))],
                        dtype=torch.int32, device=DEV)
    out = torch.full_like(q, float("nan"))
    scale = 1 / math.sqrt(hd)
    part_o = part_ml = None
    if nsplit > 1:
        slabs = work.shape[0] * 2 * nkv * nsplit * 128
        part_o = torch.full((slabs, hd), float("nan"), device=DEV)
        part_ml = torch.full((slabs, 2), float("nan"), device=DEV)
    ops().paged_attention_prefill_tcgen05(q, kc, vc, out, bt, cu, kvl, work, nq, nkv, hd, ps, scale, window, tiles,
                                          nsplit, chunk, part_o, part_ml)
    torch.cuda.synchronize()
    assert ops().gemm_error_flag(q.device) == 0
    kc, vc = torch.nan_to_num(kc), torch.nan_to_num(vc)
    ref = ref_paged_attention(q, kc, vc, tables, eot.cpu(), pos.cpu(), nq, nkv, hd, ps, scale, window)
    got = out.float().cpu().view(-1, nq, hd).double()
    assert torch.isfinite(got).all()
    assert torch.allclose(got, ref, rtol=2e-2, atol=2e-2)


def test_paged_attention_prefill_tcgen05_refuses():
    q = torch.zeros(4, 2, 64, device=DEV, dtype=torch.bfloat16)
    kc = torch.zeros(4, 2, 16, 64, device=DEV, dtype=torch.bfloat16)
    bt = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(Exception, match="attention_prefill_tcgen05"):
        ops().paged_attention_prefill_tcgen05(q, kc, kc, q.clone(), bt, z, z, z.view(1, 2), 2, 2, 64, 16, 1.0, 0)


@pytest.mark.parametrize("M, N, K", [(1, 64, 64), (8, 4096, 4096), (5, 200, 520), (8, 96, 264),
                                     (7, 5120, 1024), (8, 6144, 4096)])       # 320 and 384 blocks: the lean form
def test_gemm_skinny_with_fused_norms(M, N, K):
    """residual += x.W^T with the next norm prepared in the epilogue, then a product that consumes it."""
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    residual = torch.randn(M, N, device=DEV, generator=g) * 2
    nw = 1 + 0.1 * torch.randn(N, device=DEV, generator=g)
    eps = 1e-5
    res = residual.clone()
    xw = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    ss = torch.full(((N + 15) // 16, 8), float("nan"), device=DEV)
    ops().gemm_tn_skinny_fused(x, w1, residual=res, next_w=nw, xw_out=xw, ss_out=ss)
    new_res = residual.double() + x.double() @ w1.double().T
    assert torch.allclose(res.double(), new_res, rtol=1e-4, atol=1e-3)
    assert torch.allclose(xw.double(), new_res * nw.double(), rtol=1e-2, atol=1e-2)
    assert torch.allclose(ss.sum(0)[:M].double(), (new_res ** 2).sum(-1), rtol=1e-4)
    assert torch.all(ss[:, M:] == 0)
    # the consumer: y = rmsnorm(new_res) . W2^T through the lazily normalised input
    N2 = 48
    w2 = (torch.randn(N2, N, device=DEV, generator=g) / math.sqrt(N)).to(torch.bfloat16) if N % 8 == 0 else None
    if w2 is not None:
        y = torch.full((M, N2), float("nan"), device=DEV, dtype=torch.float32)
        ops().gemm_tn_skinny_fused(xw, w2, y, scale_parts=ss, norm_width=N, eps=eps)
        normed = new_res * torch.rsqrt((new_res ** 2).mean(-1, keepdim=True) + eps) * nw.double()
        assert torch.allclose(y.double(), normed @ w2.double().T, rtol=2e-2, atol=2e-2)
    # residual only (nothing follows)
    res2 = residual.clone()
    ops().gemm_tn_skinny_fused(x, w1, residual=res2)
    assert torch.equal(res2, res)


@pytest.mark.parametrize("M, N, K", [(9, 4096, 4096), (64, 4096, 12288), (33, 200, 520), (17, 5120, 1024), (64, 96, 264),
                                     (5, 384, 8192), (48, 136, 72), (128, 4096, 4096), (100, 200, 520),
                                     (65, 5120, 1024), (97, 24576, 136)])
def test_gemm_tcgen05_with_fused_norms(M, N, K):
    """The same fusions in the one-tile tensor-core product (9 to 128 tokens; K split over a cluster, over
    the workspace, or not at all): residual += x.W^T with the next norm prepared in the epilogue, then
    products that consume it, plain and through SwiGLU."""
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    residual = torch.randn(M, N, device=DEV, generator=g) * 2
    nw = 1 + 0.1 * torch.randn(N, device=DEV, generator=g)
    eps = 1e-5
    res = residual.clone()
    xw = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    ss = torch.full(((N + 127) // 128, 128), float("nan"), device=DEV)
    ops().gemm_tn_tcgen05_fused(x, w1, residual=res, next_w=nw, xw_out=xw, ss_out=ss)
    assert ops().gemm_error_flag(x.device) == 0
    new_res = residual.double() + x.double() @ w1.double().T
    assert torch.allclose(res.double(), new_res, rtol=1e-4, atol=1e-3)
    assert torch.allclose(xw.double(), new_res * nw.double(), rtol=1e-2, atol=1e-2)
    assert torch.allclose(ss[:, :M].sum(0).double(), (new_res ** 2).sum(-1), rtol=1e-4)
    # what the consumers compute: the next norm's input as the producer stored it (rounded to bfloat16), times
    # the weights, scaled per token by 1 / RMS of the float32 residual
    inv_rms = torch.rsqrt((new_res ** 2).mean(-1, keepdim=True) + eps)
    lazy = xw.double() * inv_rms
    assert torch.allclose(lazy, new_res * inv_rms * nw.double(), rtol=1e-2, atol=1e-2)     # = rmsnorm(new_res)
    if N % 8 == 0:
        for N2 in (48, 1000):
            w2 = (torch.randn(N2, N, device=DEV, generator=g) / math.sqrt(N)).to(torch.bfloat16)
            y = torch.full((M, N2), float("nan"), device=DEV, dtype=torch.float32)
            ops().gemm_tn_tcgen05_fused(xw, w2, y, scale_parts=ss, norm_width=N, eps=eps)
            assert torch.allclose(y.double(), lazy @ w2.double().T, rtol=1e-4, atol=1e-3)
        w3 = (torch.randn(320, N, device=DEV, generator=g) * 2 / math.sqrt(N)).to(torch.bfloat16)
        h = torch.full((M, 160), float("nan"), device=DEV, dtype=torch.bfloat16)
        ops().gemm_tn_tcgen05_fused(xw, w3, h, swiglu8=True, scale_parts=ss, norm_width=N, eps=eps)
        full = (lazy @ w3.double().T).view(M, 20, 2, 8)
        ref = (torch.nn.functional.silu(full[:, :, 0]) * full[:, :, 1]).reshape(M, 160)
        assert torch.allclose(h.double(), ref, rtol=1e-2, atol=1e-3)          # the output's rounding to bfloat16
    # residual only (nothing follows): the same bits
    res2 = residual.clone()
    ops().gemm_tn_tcgen05_fused(x, w1, residual=res2)
    assert torch.equal(res2, res)
    assert ops().gemm_error_flag(x.device) == 0


_FALLBACK_FORMS = r"""
import math, sys, torch
from safetyraise_lmengine_b200.kernels import ops
dev = "cuda:0"
for M, N, K, splits in [(2048, 6144, 1024, 1), (900, 6144, 2048, 1), (512, 6000, 2048, 1), (64, 4096, 4096, 4),
                        (33, 512, 2048, 3), (128, 4096, 12288, 4), (20, 136, 8192, 12)]:
    g = torch.Generator(device=dev).manual_seed(M + N)
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=dev, generator=g).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=dev)
    ops.gemm_tn_tcgen05(a, w, out, splits=splits)
    out2 = torch.full((M, N), float("nan"), device=dev)
    ops.gemm_tn_tcgen05(a, w, out2, splits=splits)
    ref = a.float() @ w.float().T
    assert ops.gemm_error_flag(a.device) == 0
    assert torch.allclose(out, ref, rtol=1e-4, atol=2e-4 * math.sqrt(K)), (M, N, K, splits)
    assert torch.equal(out, out2), (M, N, K, splits)
print("fallback forms agree")
"""


def test_gemm_tcgen05_forms_behind_the_switches():
    """The forms that the defaults no longer reach: one SM per tile of 128 x 256 (no pairs), whole tiles only
    (no dealing), K splits through the workspace (no cluster).  The switches are read once per process,
    hence a process of its own."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, SRLM_GEMM_PAIR="0", SRLM_GEMM_STREAMK="0", SRLM_GEMM_CLUSTER="0",
               PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    done = subprocess.run([sys.executable, "-c", _FALLBACK_FORMS], env=env, capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 0 and "fallback forms agree" in done.stdout, done.stdout[-2000:] + done.stderr[-2000:]


def test_products_of_random_sizes_through_the_dispatcher():
    """Token counts, widths and depths drawn at random (a fixed seed) through ``ops.gemm`` and, up to 128
    tokens, through the form with the residual and the next norm inside: whatever tile, split and ring the
    plans pick for a size, the result is the float32 reference's."""
    import random
    rnd = random.Random(0)
    g = torch.Generator(device=DEV).manual_seed(1)
    done = 0
    while done < 150:
        M = rnd.choice([1, 2, 3, 5, 8, 9, 12, 16, 17, 24, 31, 32, 33, 48, 63, 64, 65, 96, 127, 128, 129, 200, 256, 257,
                        400, 512, 700])
        N = rnd.choice([8, 16, 24, 96, 100, 128, 136, 264, 1000, 2048, 4096, 5120, 6144, 7168, 9000, 24576])
        K = 8 * rnd.choice([1, 3, 8, 9, 16, 33, 64, 72, 128, 257, 512, 640, 1024, 1536, 2176])
        if M * N > 6e6 or N * K > 7e7:
            continue
        done += 1
        a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
        out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.float32)
        ops().gemm(a, w, out)
        ref = a.float() @ w.float().T
        assert torch.allclose(out, ref, rtol=1e-4, atol=2e-4 * math.sqrt(K)), (M, N, K)
        if M <= 128 and N % 8 == 0:
            res = torch.randn(M, N, device=DEV, generator=g)
            got = res.clone()
            xw = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
            ss = torch.zeros((N + 127) // 128, 128, device=DEV)
            ops().gemm_tn_tcgen05_fused(a, w, residual=got, next_w=torch.ones(N, device=DEV), xw_out=xw, ss_out=ss)
            want = res.double() + a.double() @ w.double().T
            assert torch.allclose(got.double(), want, rtol=1e-4, atol=1e-3), (M, N, K)
            assert torch.allclose(ss[:, :M].sum(0).double(), (want ** 2).sum(-1), rtol=1e-4, atol=1e-4), (M, N, K)
    assert ops().gemm_error_flag(torch.device(DEV)) == 0

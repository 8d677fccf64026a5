"""Each CUDA kernel alone against a plain PyTorch float32 reference of the same
operation, at sizes other than the engine's tiny models (widths and vocabularies that are
no power of two, head sizes in steps of 16, any number of heads and groups)."""
import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def dev():
    from vosti_b200 import ops
    device = torch.device("cuda:0")
    ops.require_device(device)
    return device


@pytest.fixture()
def status(dev):
    return torch.zeros(1, dtype=torch.int32, device=dev)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(80, 331), (7, 19), (4096, 1000)])
def test_embedding(dev, status, dtype, hidden, vocab):
    from vosti_b200 import ops
    table = torch.randn(vocab, hidden, device=dev).to(dtype)
    ids = torch.randint(0, vocab, (37,), device=dev, dtype=torch.int32)
    out = ops.embedding(ids, table, status)
    assert torch.equal(out, table[ids.long()]) and status.item() == 0
    bad = ids.clone()
    bad[3] = vocab
    out = ops.embedding(bad, table, status)
    assert status.item() == 1 and out[3].abs().max() == 0        # reported, not read


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [80, 100, 1000, 4096 + 24, 8192 + 40])   # vector and scalar paths
@pytest.mark.parametrize("weight_f32", [False, True])
def test_rmsnorm(dev, dtype, width, weight_f32):
    from vosti_b200 import ops
    x = (torch.randn(11, width, device=dev) * 3).to(dtype)
    r = torch.randn(11, width, device=dev).to(dtype)
    w = (1 + 0.1 * torch.randn(width, device=dev)).to(torch.float32 if weight_f32 else dtype)
    eps = 3e-5
    out, _ = ops.rmsnorm(x, w, eps)
    want = plain.rms_norm(x.float().cpu(), w.float().cpu(), eps)
    assert torch.allclose(out.float().cpu(), want, **tol(dtype))
    res = r.clone()
    out, new_res = ops.rmsnorm(x, w, eps, residual=res, residual_out=res)
    want_n, want_r = plain.add_rms_norm(x.float().cpu(), r.float().cpu(), w.float().cpu(), eps)
    assert new_res is res
    assert torch.allclose(res.float().cpu(), want_r, **tol(dtype))
    assert torch.allclose(out.float().cpu(), want_n, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dev, dtype):
    from vosti_b200 import ops
    gu = (torch.randn(13, 2 * 200, device=dev) * 4).to(dtype)
    out = ops.silu_mul(gu)
    g, u = gu.float()[:, :200], gu.float()[:, 200:]
    assert torch.allclose(out.float(), (g * torch.sigmoid(g) * u).to(dtype).float(), **tol(dtype))


@pytest.mark.parametrize("xdt,wdt,ydt", [(torch.float32, torch.float32, torch.float32),
                                         (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                         (torch.bfloat16, torch.bfloat16, torch.float32),
                                         (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("rows,n,k", [(1, 331, 80), (37, 200, 96), (130, 67, 1000), (5, 1, 3)])
def test_gemm_simt(dev, status, xdt, wdt, ydt, rows, n, k):
    from vosti_b200 import ops
    x = torch.randn(rows, k, device=dev).to(xdt)
    w = (torch.randn(n, k, device=dev) / math.sqrt(k)).to(wdt)
    y = ops.gemm_simt(x, w, status, out_dtype=ydt)
    want = x.double() @ w.double().T
    assert y.dtype == ydt and torch.allclose(y.double(), want, **tol(ydt))
    index = torch.randint(0, rows, (9,), device=dev, dtype=torch.int32)
    y = ops.gemm_simt(x, w, status, out_dtype=ydt, row_index=index)
    assert torch.allclose(y.double(), want[index.long()], **tol(ydt)) and status.item() == 0


def test_gemm_simt_is_true_float32_and_row_independent(dev, status):
    """No reduced-precision matrix mode: values that TF32 would round survive; and a row's
    result does not depend on the other rows of the launch."""
    from vosti_b200 import ops
    k = 64
    x = torch.zeros(3, k, device=dev)
    x[:, 0] = 1.0 + 2.0 ** -20                                   # needs more than 10 mantissa bits
    w = torch.zeros(2, k, device=dev)
    w[:, 0] = 1.0
    y = ops.gemm_simt(x, w, status)
    assert y[0, 0].item() == 1.0 + 2.0 ** -20
    a = torch.randn(70, 300, device=dev)
    b = torch.randn(130, 300, device=dev)
    full = ops.gemm_simt(a, b, status)
    for r in (0, 33, 69):
        assert torch.equal(ops.gemm_simt(a[r:r + 1].contiguous(), b, status)[0], full[r])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [19, 150])          # few tokens: a warp per head; many: blocks streaming over tokens
@pytest.mark.parametrize("nq,nkv,d,use_norm,use_rope", [(6, 3, 48, True, True), (4, 4, 16, False, True),
                                                         (5, 1, 128, True, False), (8, 2, 256, True, True),
                                                         (9, 3, 64, True, True), (32, 8, 128, True, True)])
def test_qkv_post(dev, status, dtype, T, nq, nkv, d, use_norm, use_rope):
    _check_qkv_post(dev, status, dtype, T, nq, nkv, d, use_norm, use_rope)


@pytest.mark.parametrize("nq,nkv,d,use_norm,use_rope", [(5, 1, 128, True, False), (8, 2, 256, True, True),
                                                         (9, 3, 64, True, True), (32, 8, 128, True, True)])
def test_qkv_post_streams_over_more_tokens_than_its_ring_holds(dev, status, nq, nkv, d, use_norm, use_rope):
    """3,000 tokens: every block of the streaming kernel takes more tokens than its ring of buffers
    holds, so the buffers are used again."""
    _check_qkv_post(dev, status, torch.bfloat16, 3000, nq, nkv, d, use_norm, use_rope)


def _check_qkv_post(dev, status, dtype, T, nq, nkv, d, use_norm, use_rope):
    from vosti_b200 import ops
    slots_total, eps, theta = 2 * T + 26, 2e-6, 50000.0
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=dev).to(dtype)
    qw = (1 + 0.1 * torch.randn(d, device=dev)).to(dtype) if use_norm else None
    kw = (1 + 0.1 * torch.randn(d, device=dev)).to(dtype) if use_norm else None
    positions = torch.randint(0, 500, (T,), device=dev, dtype=torch.int32)
    cos = sin = None
    if use_rope:
        c, s = plain.rope_tables(torch.arange(500), d, theta)
        cos, sin = c.to(dev).contiguous(), s.to(dev).contiguous()
    slots = torch.randperm(slots_total, device=dev)[:T].to(torch.int32)
    slots[4] = -1                                               # a skipped row
    k_cache = torch.full((slots_total, nkv, d), float("nan"), device=dev).to(dtype)
    v_cache = torch.full((slots_total, nkv, d), float("nan"), device=dev).to(dtype)
    q = ops.qkv_post(qkv, k_cache, v_cache, nq=nq, nkv=nkv, head_dim=d, q_norm_w=qw, k_norm_w=kw, eps=eps,
                     cos=cos, sin=sin, positions=positions, slot_mapping=slots, status=status)
    f = qkv.float().cpu()
    qr = f[:, :nq * d].view(T, nq, d)
    kr = f[:, nq * d:(nq + nkv) * d].view(T, nkv, d)
    vr = f[:, (nq + nkv) * d:].view(T, nkv, d)
    if use_norm:
        qr, kr = plain.head_rms_norm(qr, qw.float().cpu(), eps), plain.head_rms_norm(kr, kw.float().cpu(), eps)
    if use_rope:
        c, s = plain.rope_tables(positions.cpu(), d, theta)
        qr, kr = plain.apply_rope(qr, c, s), plain.apply_rope(kr, c, s)
    assert torch.allclose(q.float().cpu().view(T, nq, d), qr, **tol(dtype))
    keep = [t for t in range(T) if t != 4]
    sl = slots.long().cpu()[keep]
    assert torch.allclose(k_cache.float().cpu()[sl], kr[keep], **tol(dtype))
    assert torch.equal(v_cache.float().cpu()[sl], vr[keep].to(dtype).float())
    untouched = torch.ones(slots_total, dtype=torch.bool)
    untouched[sl] = False
    assert torch.isnan(k_cache.float().cpu()[untouched]).all()  # nothing else was written
    assert status.item() == 0
    slots[0] = slots_total
    ops.qkv_post(qkv, k_cache, v_cache, nq=nq, nkv=nkv, head_dim=d, q_norm_w=qw, k_norm_w=kw, eps=eps,
                 cos=cos, sin=sin, positions=positions, slot_mapping=slots, status=status)
    assert status.item() & 2


def paged_case(dev, dtype, lens_q, lens_k, nq, nkv, d, page, poison=True, seed=0):
    """Random requests with their keys scattered over shuffled pages; unused cache is NaN."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens_q)
    pages_of = [(k + page - 1) // page for k in lens_k]
    num_pages = sum(pages_of) + 3
    order = torch.randperm(num_pages, generator=g).tolist()
    fill = float("nan") if poison else 0.0
    k_cache = torch.full((num_pages * page, nkv, d), fill)
    v_cache = torch.full((num_pages * page, nkv, d), fill)
    max_pages = max(pages_of)
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    ks, vs, qs, positions, request_of = [], [], [], [], []
    for b in range(B):
        mine = [order.pop() for _ in range(pages_of[b])]
        table[b, :len(mine)] = torch.tensor(mine, dtype=torch.int32)
        k = torch.randn(lens_k[b], nkv, d, generator=g).to(dtype).float()
        v = torch.randn(lens_k[b], nkv, d, generator=g).to(dtype).float()
        for j in range(lens_k[b]):
            slot = mine[j // page] * page + j % page
            k_cache[slot], v_cache[slot] = k[j], v[j]
        ks.append(k), vs.append(v)
        qs.append(torch.randn(lens_q[b], nq, d, generator=g).to(dtype).float())
        positions += list(range(lens_k[b] - lens_q[b], lens_k[b]))
        request_of += [b] * lens_q[b]
    return dict(q=torch.cat(qs), ks=ks, vs=vs, qs=qs, k_cache=k_cache, v_cache=v_cache, table=table,
                positions=torch.tensor(positions, dtype=torch.int32),
                request_of=torch.tensor(request_of, dtype=torch.int32), page=page)


def dev_cache(case, key, dev, dtype):
    """The test builds caches as [slot, kv head, d]; the kernels keep [page, kv head, offset, d]."""
    c, page = case[key], case["page"]
    return c.view(-1, page, c.shape[1], c.shape[2]).permute(0, 2, 1, 3).contiguous().to(dev, dtype)


def reference_attention(case, scale, window):
    outs = []
    for q, k, v in zip(case["qs"], case["ks"], case["vs"]):
        L, n = k.shape[0], q.shape[0]
        full_q = torch.zeros(L, q.shape[1], q.shape[2])
        full_q[L - n:] = q
        outs.append(plain.causal_attention(full_q, k, v, scale, window=window)[L - n:])
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,window", [(6, 3, 48, 16, 0), (4, 1, 16, 8, 0), (8, 8, 128, 16, 0),
                                                   (6, 2, 80, 4, 13), (2, 1, 256, 64, 0), (4, 2, 32, 8, 40)])
def test_attention_simt(dev, status, dtype, nq, nkv, d, page, window):
    from vosti_b200 import ops
    lens_k = [1, 33, 64, 130, 17, 95]
    lens_q = [1, 33, 1, 7, 2, 1]
    case = paged_case(dev, dtype, lens_q, lens_k, nq, nkv, d, page)
    scale = 0.37 * d ** -0.5
    out = ops.attention_simt(case["q"].to(dev, dtype), dev_cache(case, "k_cache", dev, dtype), dev_cache(case, "v_cache", dev, dtype),
                             positions=case["positions"].to(dev), request_of=case["request_of"].to(dev),
                             block_table=case["table"].to(dev), page_size=page, nq=nq, nkv=nkv, head_dim=d,
                             scale=scale, window=window, status=status)
    want = reference_attention(case, scale, window)
    assert torch.isfinite(out).all(), "a masked or unused (NaN) cache entry was read"
    assert torch.allclose(out.float().cpu(), want, **tol(dtype)) and status.item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dev, status, dtype):
    """One key among hundreds is made to stand out (query and key scaled); the output must be
    that key's value. Placed at a page's first and last slot and at the window's edge."""
    from vosti_b200 import ops
    nq, nkv, d, page = 2, 1, 32, 16
    for L, far, window in [(400, 0, 0), (400, 15, 0), (400, 16, 0), (400, 383, 0), (400, 399, 0),
                           (400, 300, 100), (400, 299, 100)]:
        case = paged_case(dev, dtype, [1], [L], nq, nkv, d, page, seed=L + far)
        direction = torch.nn.functional.normalize(torch.randn(d), dim=0)
        case["q"][0, :, :] = 40.0 * direction
        slot = int(case["table"][0, far // page]) * page + far % page
        case["k_cache"][slot, 0] = (40.0 * direction).to(dtype).float()
        marker = torch.full((d,), 3.0)
        case["v_cache"][slot, 0] = marker
        out = ops.attention_simt(case["q"].to(dev, dtype), dev_cache(case, "k_cache", dev, dtype),
                                 dev_cache(case, "v_cache", dev, dtype), positions=case["positions"].to(dev),
                                 request_of=case["request_of"].to(dev), block_table=case["table"].to(dev),
                                 page_size=page, nq=nq, nkv=nkv, head_dim=d, scale=1.0, window=window, status=status)
        visible = window == 0 or far > L - 1 - window
        if visible:
            assert torch.allclose(out.float().cpu()[0], marker.expand(nq, d), atol=2e-2), (L, far, window)
        else:
            assert (out.float().cpu()[0] - 3.0).abs().mean() > 0.5, (L, far, window)


def test_attention_refuses_sizes_it_cannot_do(dev, status):
    from vosti_b200 import ops
    q = torch.zeros(1, 2 * 24, device=dev)
    cache = torch.zeros(16, 1, 24, device=dev)
    with pytest.raises(ops.KernelError, match="multiple of 16"):
        ops.attention_simt(q, cache, cache, positions=torch.zeros(1, dtype=torch.int32, device=dev),
                           request_of=torch.zeros(1, dtype=torch.int32, device=dev),
                           block_table=torch.zeros(1, 1, dtype=torch.int32, device=dev), page_size=16, nq=2,
                           nkv=1, head_dim=24, scale=1.0, window=0, status=status)


def test_sampling(dev):
    from vosti_b200 import ops
    vocab = 1531
    logits = torch.randn(6, vocab, device=dev) * 2
    logits[1, 700] = logits[1, 20] = 50.0                        # a tie: the lowest index wins
    assert ops.sample(logits).tolist() == [int(torch.argmax(r)) if i != 1 else 20 for i, r in enumerate(logits.cpu())]
    temps = torch.tensor([0.0, 0.0, 0.7, 1.0, 1.3, 0.7], device=dev)
    hits = 0
    for index in range(40):
        seeds = torch.tensor([3, 3, 5, 2 ** 40 + 7, 11, 6], dtype=torch.int64, device=dev)
        counters = torch.full((6,), index, dtype=torch.int64, device=dev)
        got = ops.sample(logits, temps, seeds, counters).tolist()
        assert got[0] == int(torch.argmax(logits[0])) and got[1] == 20
        for row in range(2, 6):
            t = float(temps[row])
            w = torch.exp((logits[row].double().cpu() - logits[row].double().cpu().max()) / t)
            cdf = torch.cumsum(w, 0)
            u = plain.uniform(int(seeds[row]), index) * float(cdf[-1])
            low = float(cdf[got[row] - 1]) if got[row] > 0 else 0.0
            slack = 1e-5 * float(cdf[-1])
            assert low - slack <= u <= float(cdf[got[row]]) + slack, (row, index)
            hits += got[row] == plain.sample(logits[row].cpu(), t, int(seeds[row]), index)
    assert hits >= 155                                           # equal to the plain sampler but for rounding at an edge
    assert ops.sample(logits, temps, seeds, counters).tolist() == got      # same state, same token


# ---------------------------------------------------------------- tensor-core product
@pytest.mark.parametrize("tokens", [1, 7, 33, 64, 100, 129, 300, 1100])
@pytest.mark.parametrize("features,k", [(64, 64), (200, 80), (331, 96), (200, 320), (72, 448), (4096, 1000), (1536, 4096),
                                        (152, 12288)])
def test_gemm_tc(dev, status, tokens, features, k):
    from vosti_b200 import ops
    assert ops.gemm_tc_supported(features, k)
    x = torch.randn(tokens, k, device=dev).bfloat16()
    w = (torch.randn(features, k, device=dev) / math.sqrt(k)).bfloat16()
    want = x.double() @ w.double().T
    y32 = ops.gemm_tc(x, w, status, out_dtype=torch.float32)
    assert torch.allclose(y32.double(), want, atol=2e-4, rtol=2e-4), (y32.double() - want).abs().max()
    y16 = ops.gemm_tc(x, w, status)
    assert y16.dtype == torch.bfloat16 and torch.allclose(y16.double(), want, atol=2e-2, rtol=2e-2)
    assert torch.equal(y16, y32.bfloat16())                       # one rounding, at the store
    assert status.item() == 0


def test_gemm_tc_refuses_what_it_cannot_do(dev, status):
    from vosti_b200 import ops
    assert not ops.gemm_tc_supported(64, 48) and not ops.gemm_tc_supported(64, 100)
    with pytest.raises(ops.KernelError):
        ops.gemm_tc(torch.zeros(4, 100, device=dev).bfloat16(), torch.zeros(8, 100, device=dev).bfloat16(), status)


@pytest.mark.parametrize("tokens", [3, 70, 400])
@pytest.mark.parametrize("inter,k", [(128, 64), (208, 96), (12288 // 8, 4096)])
def test_gemm_tc_fused_silu_mul(dev, status, tokens, inter, k):
    """SiLU(gate)*up in the epilogue, with the weight rows in blocks of 16 gate and 16 up
    rows, against the unfused order of operations."""
    from vosti_b200 import ops
    x = torch.randn(tokens, k, device=dev).bfloat16()
    gate = (torch.randn(inter, k, device=dev) / math.sqrt(k)).bfloat16()
    up = (torch.randn(inter, k, device=dev) / math.sqrt(k)).bfloat16()
    blocks = torch.stack([gate.view(-1, 16, k), up.view(-1, 16, k)], dim=1).reshape(2 * inter, k).contiguous()
    y = ops.gemm_tc(x, blocks, status, swiglu=True)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = g * torch.sigmoid(g) * u
    assert y.shape == (tokens, inter) and torch.allclose(y.double(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("tokens", [5, 70, 300])
@pytest.mark.parametrize("features,k", [(1000, 1000), (384, 64), (4096 + 128, 4096), (96, 200), (130, 320)])
def test_gemm_tc_tile_packed_weight_gives_the_same_bits(dev, status, tokens, features, k):
    """A weight stored tile by tile (zero-padded to whole tiles) multiplies to the same bits
    as the row-major weight, in both kernels, with split K and with the fused SiLU epilogue."""
    from vosti_b200 import ops
    x = torch.randn(tokens, k, device=dev).bfloat16()
    w = (torch.randn(features, k, device=dev) / 16).bfloat16()
    packed = ops.PackedWeight(w)
    assert packed.shape == (features, k) and packed.data.shape[2:] == (128, 64)
    for out_dtype in (torch.bfloat16, torch.float32):
        assert torch.equal(ops.gemm_tc(x, w, status, out_dtype=out_dtype), ops.gemm_tc(x, packed, status, out_dtype=out_dtype))
    a = ops.materialize(ops.gemm_tc(x, w, status, allow_partial=True))      # one deferred result at a time
    b = ops.materialize(ops.gemm_tc(x, packed, status, allow_partial=True))
    assert torch.equal(a, b)
    if features % 32 == 0:
        assert torch.equal(ops.gemm_tc(x, w, status, swiglu=True), ops.gemm_tc(x, packed, status, swiglu=True))
    assert status.item() == 0


def test_gemm_tc_rows_do_not_depend_on_their_companions(dev, status):
    """Within one tile size and split count a row's bits do not depend on the other rows."""
    from vosti_b200 import ops
    k, features = 4096, 1024
    x = torch.randn(24, k, device=dev).bfloat16()
    w = (torch.randn(features, k, device=dev) / 64).bfloat16()
    full = ops.gemm_tc(x, w, status, out_dtype=torch.float32)
    for r in (0, 11, 23):
        alone = ops.gemm_tc(x[r:r + 1].contiguous(), w, status, out_dtype=torch.float32)
        assert torch.equal(alone[0], full[r])
    big = torch.randn(700, k, device=dev).bfloat16()
    full = ops.gemm_tc(big, w, status, out_dtype=torch.float32)
    part = ops.gemm_tc(big[300:600].contiguous(), w, status, out_dtype=torch.float32)
    assert torch.equal(part, full[300:600])


# ---------------------------------------------------------------- tensor-core attention
def _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, scale, window, which, kernel=None):
    """Drive the decode (one query at a time) or the portion kernel directly."""
    from vosti_b200 import ops
    q = case["q"].to(dev, torch.bfloat16)
    kc, vc = dev_cache(case, "k_cache", dev, torch.bfloat16), dev_cache(case, "v_cache", dev, torch.bfloat16)
    out = torch.full_like(q, float("nan"))
    table = case["table"].to(dev)
    common = dict(block_table=table, page_size=page, nq=nq, nkv=nkv, head_dim=d, scale=scale, window=window, status=status)
    if which == "decode":
        ops.attention_decode(q, kc, vc, out, token_list=None, count=q.shape[0], positions=case["positions"].to(dev),
                             request_of=case["request_of"].to(dev), max_kv_len=max(lens_k), **common)
    else:
        cu = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=dev)
        ops.attention_prefill(q, kc, vc, out, row_list=None, count=len(lens_q), cu_q=cu,
                              kv_len=torch.tensor(lens_k, dtype=torch.int32, device=dev), max_q_len=max(lens_q),
                              kernel=kernel, **common)
    return out


@pytest.mark.parametrize("which", ["decode", "prefill"])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(6, 3, 48, 16, 0), (4, 1, 16, 8, 0), (8, 8, 128, 16, 0),
                                                   (6, 2, 80, 4, 13), (16, 1, 256, 64, 0), (4, 2, 32, 8, 300),
                                                   (32, 8, 128, 16, 0), (12, 4, 64, 16, 77)])
def test_attention_tensor_cores(dev, status, which, nq, nkv, d, page, window):
    lens_k = [1, 33, 64, 130, 17, 95, 700, 257, 256]
    lens_q = [1, 33, 1, 7, 2, 1, 300, 1, 2] if which == "prefill" else [1, 3, 1, 4, 2, 1, 2, 1, 2]
    case = paged_case(dev, torch.bfloat16, lens_q, lens_k, nq, nkv, d, page)
    scale = 0.37 * d ** -0.5
    out = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, scale, window, which)
    want = reference_attention(case, scale, window)
    assert torch.isfinite(out).all(), "a row was not written or an unused (NaN) cache entry was read"
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), (out.float().cpu() - want).abs().max()
    assert status.item() == 0


@pytest.mark.parametrize("nq,nkv,d,page,window", [(4, 4, 128, 16, 0), (8, 4, 64, 32, 0), (16, 2, 128, 64, 0),
                                                   (16, 1, 64, 16, 45), (5, 1, 128, 16, 0), (14, 2, 64, 48, 129),
                                                   (32, 8, 128, 16, 1000)])
def test_prefill_attention_on_tcgen05(dev, status, nq, nkv, d, page, window):
    """The tensor-memory kernel against the plain formula and against the mma.sync kernel: every
    group size (also ones that do not divide 128 rows), pages of 16, 32, 48 and 64 tokens,
    windows, whole prompts and portions that continue a cached prefix."""
    from vosti_b200 import ops
    assert ops.library().vosti_attention_prefill_tc_supported(d, page)
    lens_k = [1, 33, 64, 130, 17, 95, 700, 257, 256, 1500]
    lens_q = [1, 33, 5, 7, 17, 40, 300, 129, 2, 1000]
    case = paged_case(dev, torch.bfloat16, lens_q, lens_k, nq, nkv, d, page)
    scale = 0.41 * d ** -0.5
    out = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, scale, window, "prefill", kernel="tc")
    other = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, scale, window, "prefill", kernel="mma")
    want = reference_attention(case, scale, window)
    assert torch.isfinite(out).all(), "a row was not written or an unused (NaN) cache entry was read"
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), (out.float().cpu() - want).abs().max()
    assert torch.allclose(out.float(), other.float(), atol=2e-2, rtol=2e-2)
    assert status.item() == 0


@pytest.mark.parametrize("step", [0.02, 0.2, 2.0])
def test_prefill_attention_on_tcgen05_with_a_rising_maximum(dev, status, step):
    """Scores that grow with the key index: the kernel's reference maximum is raised (and the
    running product in tensor memory scaled down) at every tile for the steep ramp, only now
    and then for the gentle ones, where exponentials above one are accumulated in between."""
    nq, nkv, d, page, L = 8, 2, 128, 16, 900
    case = paged_case(dev, torch.bfloat16, [L], [L], nq, nkv, d, page, seed=3)
    direction = torch.nn.functional.normalize(torch.randn(d), dim=0)
    case["q"][:, :, :] = (8.0 * direction + 0.1 * torch.randn(L, nq, d)).bfloat16().float()
    case["qs"][0][:] = case["q"]
    for pos in range(L):
        slot = int(case["table"][0, pos // page]) * page + pos % page
        case["ks"][0][pos] = (step * pos * direction + 0.05 * torch.randn(nkv, d)).bfloat16().float()
        case["k_cache"][slot, :] = case["ks"][0][pos]
    out = _run_tc_attention(dev, status, case, [L], [L], nq, nkv, d, page, 1.0, 0, "prefill", kernel="tc")
    want = reference_attention(case, 1.0, 0)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), want, atol=3e-2, rtol=3e-2), (out.float().cpu() - want).abs().max()


def test_prefill_attention_on_tcgen05_rows_do_not_depend_on_companions(dev, status):
    """A request's rows are the same bits whether it runs alone or beside others."""
    nq, nkv, d, page = 8, 2, 128, 16
    lens_k, lens_q = [300, 1000, 513], [300, 200, 13]
    case = paged_case(dev, torch.bfloat16, lens_q, lens_k, nq, nkv, d, page)
    full = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, d ** -0.5, 0, "prefill", kernel="tc")
    from vosti_b200 import ops
    q = case["q"].to(dev, torch.bfloat16)
    kc, vc = dev_cache(case, "k_cache", dev, torch.bfloat16), dev_cache(case, "v_cache", dev, torch.bfloat16)
    out = torch.zeros_like(q)
    cu = torch.tensor([0, 300, 500, 513], dtype=torch.int32, device=dev)
    ops.attention_prefill(q, kc, vc, out, row_list=torch.tensor([1], dtype=torch.int32, device=dev), count=1, cu_q=cu,
                          kv_len=torch.tensor(lens_k, dtype=torch.int32, device=dev), block_table=case["table"].to(dev),
                          page_size=page, nq=nq, nkv=nkv, head_dim=d, max_q_len=200, scale=d ** -0.5, window=0,
                          status=status, kernel="tc")
    assert torch.equal(out[300:500], full[300:500]) and out[:300].abs().max() == 0 and out[500:].abs().max() == 0


@pytest.mark.parametrize("seed", [11, 12])
def test_attention_tensor_cores_random_shapes(dev, status, seed):
    """Head counts, groups, head sizes, page sizes, windows and lengths drawn at random (twenty
    launches per seed): whatever path the dispatcher picks must agree with the plain formula."""
    import random
    rng = random.Random(seed)
    edge_lengths = [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257, 500, 1000, 2100]
    for it in range(20):
        nkv, group = rng.choice([1, 2, 3, 4, 8]), rng.choice([1, 2, 3, 4, 5, 7, 8, 16])
        nq, d = nkv * group, rng.choice([16, 32, 48, 64, 80, 96, 128, 160, 256])
        page, window = rng.choice([1, 4, 8, 16, 16, 16, 32, 48, 64]), rng.choice([0, 0, 0, 5, 33, 100, 700])
        which = rng.choice(["decode", "prefill"])
        lens_k = [rng.choice(edge_lengths) for _ in range(rng.randint(1, 5))]
        longest_q = 4 if which == "decode" else rng.choice([1, 5, 17, 64, 100, 129, 300])
        lens_q = [min(k, rng.randint(1, longest_q)) for k in lens_k]
        if d * nq * sum(lens_k) > 1.5e8:
            continue
        case = paged_case(dev, torch.bfloat16, lens_q, lens_k, nq, nkv, d, page, seed=100 * seed + it)
        scale = 0.5 * d ** -0.5
        out = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, scale, window, which)
        want = reference_attention(case, scale, window)
        what = dict(which=which, nq=nq, nkv=nkv, d=d, page=page, window=window, lens_q=lens_q, lens_k=lens_k)
        assert torch.isfinite(out).all() and status.item() == 0, what
        assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), (what, (out.float().cpu() - want).abs().max())


@pytest.mark.parametrize("which", ["decode", "prefill"])
def test_attention_tensor_cores_find_one_far_key(dev, status, which):
    nq, nkv, d, page = 8, 2, 64, 16
    for L, far, window in [(600, 0, 0), (600, 15, 0), (600, 16, 0), (600, 255, 0), (600, 256, 0), (600, 599, 0),
                           (600, 500, 100), (600, 499, 100), (600, 63, 0), (600, 64, 0)]:
        lens_q = [1] if which == "decode" else [9]
        case = paged_case(dev, torch.bfloat16, lens_q, [L], nq, nkv, d, page, seed=L + far)
        direction = torch.nn.functional.normalize(torch.randn(d), dim=0)
        case["q"][-1, :, :] = 40.0 * direction
        slot = int(case["table"][0, far // page]) * page + far % page
        case["k_cache"][slot, :] = (40.0 * direction).bfloat16().float()
        case["v_cache"][slot, :] = 3.0
        out = _run_tc_attention(dev, status, case, lens_q, [L], nq, nkv, d, page, 1.0, window, which)
        visible = window == 0 or far > L - 1 - window
        last = out.float().cpu()[-1]
        if visible:
            assert torch.allclose(last, torch.full_like(last, 3.0), atol=3e-2), (L, far, window)
        else:
            assert (last - 3.0).abs().mean() > 0.5, (L, far, window)


@pytest.mark.parametrize("segment", [None, 64, 192, 1024, 4096])
def test_attention_decode_many_tokens_and_every_segment_length(dev, status, segment, monkeypatch):
    """More work items than resident CTAs (each CTA walks over several and prefetches across
    them), requests of very different lengths, and segment lengths from one tile per warp to
    one segment per request."""
    if segment is not None:
        monkeypatch.setenv("VOSTI_DECODE_SEGMENT", str(segment))
    nq, nkv, d, page = 8, 2, 128, 16
    generator = torch.Generator().manual_seed(7)
    lens_k = [int(x) for x in torch.randint(1, 3000, (90,), generator=generator)] + [1, 16, 17, 64, 65, 4095, 4096, 4097]
    lens_q = [1] * len(lens_k)
    case = paged_case(dev, torch.bfloat16, lens_q, lens_k, nq, nkv, d, page)
    scale = d ** -0.5
    out = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, scale, 0, "decode")
    want = reference_attention(case, scale, 0)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), (out.float().cpu() - want).abs().max()
    assert status.item() == 0


def test_attention_decode_is_independent_of_the_batch(dev, status):
    """The same token alone and among others, and listed out of order, gives the same bits, as
    long as both launches cut the keys into segments of the same length (the length is a
    function of the number of tokens and the longest context of a launch, not of their contents)."""
    from vosti_b200 import ops
    nq, nkv, d, page = 8, 2, 128, 16
    lens_k = [300, 1000, 40, 513]
    case = paged_case(dev, torch.bfloat16, [1, 1, 1, 1], lens_k, nq, nkv, d, page)
    full = _run_tc_attention(dev, status, case, [1] * 4, lens_k, nq, nkv, d, page, d ** -0.5, 0, "decode")
    q = case["q"].to(dev, torch.bfloat16)
    kc, vc = dev_cache(case, "k_cache", dev, torch.bfloat16), dev_cache(case, "v_cache", dev, torch.bfloat16)
    out = torch.zeros_like(q)
    listed = torch.tensor([3, 1], dtype=torch.int32, device=dev)
    keys = ops.library().vosti_attention_decode_segment_keys
    assert keys(4, nq, nkv, d, 1000) == keys(2, nq, nkv, d, 1000)
    ops.attention_decode(q, kc, vc, out, token_list=listed, count=2, positions=case["positions"].to(dev),
                         request_of=case["request_of"].to(dev), block_table=case["table"].to(dev), page_size=page,
                         nq=nq, nkv=nkv, head_dim=d, max_kv_len=1000, scale=d ** -0.5, window=0, status=status)
    assert torch.equal(out[3], full[3]) and torch.equal(out[1], full[1]) and out[0].abs().max() == 0


def test_deferred_split_sums_feed_the_norm_and_the_head_kernel(dev, status):
    """A split-K product may hand its unsummed splits to the fused add + RMSNorm or to the
    head-norm / rotation kernel; the results equal the unfused order of operations."""
    from vosti_b200 import ops
    tokens, k, width = 8, 4096, 1024
    x = torch.randn(tokens, k, device=dev).bfloat16()
    w = (torch.randn(width, k, device=dev) / 64).bfloat16()
    res = torch.randn(tokens, width, device=dev).bfloat16()
    nw = (1 + 0.1 * torch.randn(width, device=dev)).bfloat16()
    deferred = ops.gemm_tc(x, w, status, allow_partial=True)
    assert isinstance(deferred, ops.PartialSum) and deferred.splits > 1
    assert torch.equal(deferred.materialize(), ops.gemm_tc(x, w, status))
    deferred = ops.gemm_tc(x, w, status, allow_partial=True)
    r1 = res.clone()
    normed, _ = ops.rmsnorm(deferred, nw, 1e-6, residual=r1, residual_out=r1)
    y = x.double() @ w.double().T
    h = y + res.double()
    want = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + 1e-6) * nw.double()
    assert torch.allclose(r1.double(), h, atol=2e-2, rtol=2e-2) and torch.allclose(normed.double(), want, atol=3e-2, rtol=3e-2)
    plain_norm, _ = ops.rmsnorm(ops.gemm_tc(x, w, status, allow_partial=True), nw, 1e-6)
    want = y * torch.rsqrt((y * y).mean(-1, keepdim=True) + 1e-6) * nw.double()
    assert torch.allclose(plain_norm.double(), want, atol=3e-2, rtol=3e-2)
    # a stale deferred result is refused
    stale = ops.gemm_tc(x, w, status, allow_partial=True)
    ops.gemm_tc(x, w, status)
    with pytest.raises(ops.KernelError, match="overwrote"):
        stale.materialize()
    # the head kernel: same q and cache as from the summed projection
    nq, nkv, d = 4, 2, 128
    w2 = (torch.randn((nq + 2 * nkv) * d, k, device=dev) / 64).bfloat16()
    kc1, vc1 = torch.zeros(32, nkv, d, device=dev).bfloat16(), torch.zeros(32, nkv, d, device=dev).bfloat16()
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    qw = torch.ones(d, device=dev).bfloat16()
    c, s_ = plain.rope_tables(torch.arange(64), d, 1e4)
    args = dict(nq=nq, nkv=nkv, head_dim=d, q_norm_w=qw, k_norm_w=qw, eps=1e-6, cos=c.to(dev), sin=s_.to(dev),
                positions=torch.arange(tokens, dtype=torch.int32, device=dev),
                slot_mapping=torch.arange(tokens, dtype=torch.int32, device=dev), status=status)
    q1 = ops.qkv_post(ops.gemm_tc(x, w2, status), kc1, vc1, **args)
    q2 = ops.qkv_post(ops.gemm_tc(x, w2, status, allow_partial=True), kc2, vc2, **args)
    assert torch.allclose(q1.float(), q2.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(kc1.float(), kc2.float(), atol=2e-2, rtol=2e-2) and torch.allclose(vc1.float(), vc2.float(), atol=2e-2)


@pytest.mark.parametrize("pairs", ["1", "0"])
def test_gemm_tc_for_many_tokens_gives_the_bits_of_the_unsplit_narrow_kernel(pairs):
    """Both forms of the product for many tokens, on pairs of SMs (tcgen05 cta_group::2, the
    default) and on single SMs (VOSTI_GEMM_PAIR=0, read when the library is loaded, hence a
    process of its own), give the bits of the unsplit kernel for up to 128 tokens: row-major and
    tile-packed weights, every epilogue, edges in tokens, features and K, an odd number of
    k-blocks."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    script = r'''
import sys, torch
from vosti_b200 import ops
dev = torch.device("cuda:0")
status = torch.zeros(1, dtype=torch.int32, device=dev)
ops.set_fixed_order(True)
torch.manual_seed(0)
for (T, f, k) in [(300, 512, 256), (129, 1000, 200), (1100, 4096 + 160, 1024), (640, 1536, 4096), (257, 200, 320)]:
    w = (torch.randn(f, k, device=dev) / 8).bfloat16()
    x = torch.randn(T, k, device=dev).bfloat16()
    for W in (w, ops.PackedWeight(w)):
        for kw in (dict(), dict(out_dtype=torch.float32)) + ((dict(swiglu=True),) if f % 32 == 0 else ()):
            got = ops.gemm_tc(x, W, status, **kw)
            want = torch.cat([ops.gemm_tc(x[i:i + 128].contiguous(), W, status, **kw) for i in range(0, T, 128)])
            assert torch.equal(got, want), (T, f, k, kw)
assert status.item() == 0
print("pairs ok")
'''
    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, VOSTI_GEMM_PAIR=pairs, PYTHONPATH=str(root))
    done = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "pairs ok" in done.stdout, done.stderr[-2000:]


# ---------------------------------------------------------------- the real vocabulary
REAL_VOCAB = 151936      # the family's vocabulary: 1,187 feature tiles of 128, no power of two


def test_head_product_sampling_and_embedding_at_the_real_vocabulary(dev, status):
    """The output head on the tensor cores (float32 epilogue) and on the CUDA cores, the
    sampler and the embedding at 151,936 rows, each against a float64 reference."""
    from vosti_b200 import ops
    hidden = 1024
    gen = torch.Generator(device=dev).manual_seed(5)
    w = (torch.randn(REAL_VOCAB, hidden, device=dev, generator=gen) / math.sqrt(hidden)).bfloat16()
    x = torch.randn(9, hidden, device=dev, generator=gen).bfloat16()
    want = torch.cat([x.double() @ w[i:i + 16384].double().T for i in range(0, REAL_VOCAB, 16384)], dim=1)
    # a logit that must win although it sits in the last, partial feature tile
    last = REAL_VOCAB - 3
    for packed in (False, True):
        weight = ops.PackedWeight(w) if packed else w
        logits = ops.gemm_tc(x, weight, status, out_dtype=torch.float32)
        assert logits.shape == (9, REAL_VOCAB)
        assert torch.allclose(logits.double(), want, atol=3e-4, rtol=3e-4), (logits.double() - want).abs().max()
    narrow = ops.gemm_simt(x.float()[:3], w.float()[:, :], status, out_dtype=torch.float32)
    assert torch.allclose(narrow.double(), want[:3], atol=1e-4, rtol=1e-4)
    assert ops.sample(logits).tolist() == want.argmax(-1).tolist() or \
        all(float(want[r].max() - want[r, t]) < 1e-3 for r, t in enumerate(ops.sample(logits).tolist()))
    logits[4, last] = 100.0
    logits[5, 0] = logits[5, last] = 90.0                       # a tie across the whole width: the lowest index
    got = ops.sample(logits).tolist()
    assert got[4] == last and got[5] == 0
    temps = torch.tensor([0.0, 0.8, 1.0, 0.5, 0.7, 0.7, 1.5, 0.9, 1.1], device=dev)
    seeds = torch.arange(9, dtype=torch.int64, device=dev) + 100
    for index in (0, 1, 2):
        counters = torch.full((9,), index, dtype=torch.int64, device=dev)
        drawn = ops.sample(logits, temps, seeds, counters).tolist()
        assert drawn[0] == got[0] and drawn[4] == last          # greedy row; a row with one overwhelming logit
        for row in (1, 2, 3, 6, 7, 8):
            t = float(temps[row])
            weights = torch.exp((logits[row].double() - logits[row].double().max()) / t)
            cdf = torch.cumsum(weights, 0).cpu()
            u = plain.uniform(int(seeds[row]), index) * float(cdf[-1])
            low = float(cdf[drawn[row] - 1]) if drawn[row] > 0 else 0.0
            slack = 2e-5 * float(cdf[-1])
            assert low - slack <= u <= float(cdf[drawn[row]]) + slack, (row, index)
    ids = torch.tensor([0, last, REAL_VOCAB - 1, 77777, 151935 - 128], dtype=torch.int32, device=dev)
    assert torch.equal(ops.embedding(ids, w, status), w[ids.long()])
    assert status.item() == 0
    ops.embedding(torch.tensor([REAL_VOCAB], dtype=torch.int32, device=dev), w, status)
    assert status.item() == 1                                   # one past the end is reported, not read
    status.zero_()


@pytest.mark.parametrize("dtype", DTYPES)
def test_affine_rows(dev, dtype):
    """cap(x * scale + bias) from a float32 product, rounded once."""
    from vosti_b200 import ops
    x = torch.randn(7, 1531, device=dev) * 4
    bias = torch.randn(1531, device=dev)
    for scale, cap, b in [(1.0, 0.0, bias), (0.5, 3.0, None), (2.0, 5.0, bias.bfloat16()), (1.0, 0.0, None)]:
        want = x.double() * scale + (0 if b is None else b.double())
        if cap > 0:
            want = cap * torch.tanh(want / cap)
        got = ops.affine_rows(x.clone(), bias=b, scale=scale, softcap=cap, out_dtype=dtype)
        assert got.dtype == dtype
        if dtype == torch.float32:
            assert torch.allclose(got.double(), want, atol=1e-5, rtol=1e-5)
        else:
            assert torch.equal(got, want.float().bfloat16()) or torch.allclose(got.double(), want, atol=4e-2, rtol=1e-2)
    with pytest.raises(ops.KernelError):
        ops.affine_rows(x.bfloat16())
    with pytest.raises(ops.KernelError):
        ops.affine_rows(x, bias=bias[:-1])


def test_split_sums_wider_than_the_fused_norm_are_summed_first(dev, status):
    """The norm that adds a product's K splits keeps a row in shared memory; a wider row is
    summed by the reduction kernel first and normed by the plain kernel, instead of refused."""
    from vosti_b200 import ops
    width, splits = 24576 + 512, 3
    pieces = torch.randn(splits, 4, width, device=dev)
    residual = torch.randn(4, width, device=dev).bfloat16()
    weight = (1 + 0.1 * torch.randn(width, device=dev)).bfloat16()
    # (the product's own split rule never splits so wide a result; the sums are handed over by hand)
    partial = ops.PartialSum(pieces, splits, 4, width, torch.bfloat16, status)
    assert partial.width > ops.RMSNORM_PARTIAL_MAX_WIDTH
    res = residual.clone()
    out, new_res = ops.rmsnorm(partial, weight, 1e-6, residual=res, residual_out=res)
    product = pieces.sum(0).bfloat16()
    want_n, want_r = plain.add_rms_norm(product.float().cpu(), residual.float().cpu(), weight.float().cpu(), 1e-6)
    assert torch.allclose(new_res.float().cpu(), want_r, atol=3e-2, rtol=3e-2)
    assert torch.allclose(out.float().cpu(), want_n, atol=3e-2, rtol=3e-2)
    assert status.item() == 0


def test_weights_requested_ahead_change_no_value(dev, status):
    """The split-summing norm with a hint (it asks for the next product's weights to be brought
    into L2 from blocks added to its launch) gives the bits it gives without one; a hint is
    taken by one launch only; what is not a tile-packed weight is no hint."""
    import ctypes
    from vosti_b200 import ops
    x = torch.randn(8, 4096, device=dev).bfloat16()
    w = (torch.randn(4096, 4096, device=dev) / 64).bfloat16()
    nxt = ops.PackedWeight((torch.randn(6144, 4096, device=dev) / 64).bfloat16())
    gamma = (1 + 0.1 * torch.randn(4096, device=dev)).bfloat16()
    residual = torch.randn(8, 4096, device=dev).bfloat16()
    outs = []
    for hint in (None, nxt, w, nxt):
        partial = ops.gemm_tc(x, w, status, allow_partial=True)
        assert isinstance(partial, ops.PartialSum)
        res = residual.clone()
        assert ops.hint_prefetch(hint) == (hint is nxt and ops.PREFETCH)
        out, new_res = ops.rmsnorm(partial, gamma, 1e-6, residual=res, residual_out=res)
        outs.append((out.clone(), new_res.clone()))
    for out, res in outs[1:]:
        assert torch.equal(out, outs[0][0]) and torch.equal(res, outs[0][1])
    lib = ops.library()
    assert lib.vosti_hint_prefetch(ctypes.c_void_p(nxt.data.data_ptr() + 8), ctypes.c_longlong(1 << 20)) != 0
    assert b"16-byte" in lib.vosti_last_error()
    assert lib.vosti_hint_prefetch(None, ctypes.c_longlong(0)) == 0
    torch.cuda.synchronize()
    assert status.item() == 0


def test_sampling_with_the_state_in_request_slots(dev, status):
    """The sampler reads (temperature, seed, index) from each row's slot, draws what the array
    form draws for the same state, advances the index in the slot and notes the position; a slot
    outside the table is reported and sampled greedily."""
    from vosti_b200 import ops
    from vosti_b200.sampling import sampler_state_words
    vocab, rows, num_slots = 1531, 5, 9
    logits = torch.randn(rows, vocab, device=dev) * 2
    slot_of = [7, 2, 0, 8, 4]
    temps, seeds, start = [0.0, 0.7, 1.0, 1.3, 0.7], [3, 5, 2 ** 40 + 7, 11, 6], [0, 4, 9, 1, 30]
    table = torch.zeros(num_slots, 4, dtype=torch.int64, device=dev)
    for slot, t, s, i in zip(slot_of, temps, seeds, start):
        table[slot] = torch.tensor(sampler_state_words(t, s, i), dtype=torch.int64)
    untouched = table[[1, 3, 5, 6]].clone()
    slots = torch.tensor(slot_of, dtype=torch.int32, device=dev)
    positions = torch.tensor([40, 41, 42, 43, 44], dtype=torch.int32, device=dev)
    for step in range(3):
        got = ops.sample_slots(logits, slots, table, positions + step, status).tolist()
        want = ops.sample(logits, torch.tensor(temps, device=dev), torch.tensor(seeds, dtype=torch.int64, device=dev),
                          torch.tensor([i + step for i in start], dtype=torch.int64, device=dev)).tolist()
        assert got == want
        for row, slot in enumerate(slot_of):
            assert table[slot, 2].item() == start[row] + step + 1 and table[slot, 3].item() == 40 + row + step
            assert table[slot, 1].item() == seeds[row]
    assert torch.equal(table[[1, 3, 5, 6]], untouched) and status.item() == 0
    assert len({tuple(ops.sample_slots(logits[1:2], slots[1:2], table, None, status).tolist()) for _ in range(6)}) > 1
    bad = torch.tensor([num_slots], dtype=torch.int32, device=dev)
    assert ops.sample_slots(logits[:1], bad, table, None, status).tolist() == [int(logits[0].argmax())]
    assert status.item() == 2
    status.zero_()


@pytest.mark.parametrize("nq,nkv,d,page,window,use_norm,use_rope", [(32, 8, 128, 16, 0, True, True), (6, 3, 48, 16, 0, True, True),
                                                                     (4, 1, 16, 8, 0, False, True), (8, 8, 64, 32, 0, True, False),
                                                                     (10, 2, 128, 16, 700, True, True)])
def test_fused_decode_attention_gives_the_bits_of_its_two_kernels(dev, status, nq, nkv, d, page, window, use_norm, use_rope):
    """Head norm, rotation, cache store and attention in one kernel against the head kernel
    followed by the decode attention, from the same partial sums: the same bits in the output and
    in the caches, for requests of very different lengths, and close to the plain attention."""
    from vosti_b200 import ops
    gen = torch.Generator(device=dev).manual_seed(nq * 131 + d)
    lengths = [1, 17, 300, 1024, 1500, 2047, 33, 640]                  # keys of each request after the step
    B, heads, splits = len(lengths), nq + 2 * nkv, 5
    pages_of = [-(-n // page) for n in lengths]
    num_pages = sum(pages_of) + 3
    order = torch.randperm(num_pages - 1, generator=torch.Generator().manual_seed(1)).tolist()
    table = torch.zeros(B, max(pages_of), dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_of):
        table[b, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)
    slots = torch.tensor([int(table[b, (n - 1) // page]) * page + (n - 1) % page for b, n in enumerate(lengths)], dtype=torch.int32)
    k0 = torch.randn(num_pages, nkv, page, d, device=dev, generator=gen).bfloat16()
    v0 = torch.randn(num_pages, nkv, page, d, device=dev, generator=gen).bfloat16()
    partial = torch.randn(splits, B, heads * d, device=dev, generator=gen) * 0.6
    qw = (1 + 0.1 * torch.randn(d, device=dev, generator=gen)).bfloat16() if use_norm else None
    kw = (1 + 0.1 * torch.randn(d, device=dev, generator=gen)).bfloat16() if use_norm else None
    cos = sin = None
    if use_rope:
        cos, sin = (t.to(dev).contiguous() for t in plain.rope_tables(torch.arange(2100), d, 1e4))
    table, positions, slots = table.to(dev), positions.to(dev), slots.to(dev)
    request_of = torch.arange(B, dtype=torch.int32, device=dev)
    make = lambda: ops.PartialSum(partial, splits, B, heads * d, torch.bfloat16, status)
    common = dict(page_size=page, nq=nq, nkv=nkv, head_dim=d, scale=d ** -0.5, window=window, status=status)
    # the two kernels
    k1, v1 = k0.clone(), v0.clone()
    q = ops.qkv_post(make(), k1, v1, nq=nq, nkv=nkv, head_dim=d, page_size=page, q_norm_w=qw, k_norm_w=kw, eps=1e-6, cos=cos,
                     sin=sin, positions=positions, slot_mapping=slots, status=status)
    want = torch.empty_like(q)
    ops.attention_decode(q, k1, v1, want, token_list=None, count=B, positions=positions, request_of=request_of,
                         block_table=table, max_kv_len=2048, **common)
    # the one kernel
    k2, v2 = k0.clone(), v0.clone()
    got = ops.attention_decode_fused(make(), k2, v2, positions=positions, request_of=request_of, block_table=table,
                                     slot_mapping=slots, max_kv_len=2048, q_norm_w=qw, k_norm_w=kw, eps=1e-6, cos=cos, sin=sin,
                                     **common)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.equal(k1, k2) and torch.equal(v1, v2) and not torch.equal(k1, k0)
    assert torch.equal(got, want)
    # and the plain attention of the last request's token over its keys (no window: every key)
    if window == 0:
        b = B - 1
        n = lengths[b]
        rows = [int(table[b, i // page]) * page + i % page for i in range(n)]
        keys = k2.permute(0, 2, 1, 3).reshape(-1, nkv, d)[rows].float().cpu()
        values = v2.permute(0, 2, 1, 3).reshape(-1, nkv, d)[rows].float().cpu()
        qb = q[b].float().cpu().view(nq, d)
        ref = torch.zeros(nq, d)
        for h in range(nq):
            g = h * nkv // nq
            p = torch.softmax((keys[:, g] @ qb[h]) * d ** -0.5, 0)
            ref[h] = p @ values[:, g]
        assert torch.allclose(got[b].float().cpu().view(nq, d), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nq,nkv,d,page,window,segment", [(32, 8, 128, 16, 0, 576), (32, 8, 128, 16, 0, 192), (6, 3, 48, 16, 0, 128),
                                                           (4, 2, 256, 64, 0, 256), (12, 4, 64, 32, 77, 128),
                                                           (10, 2, 128, 48, 700, 384), (8, 8, 64, 16, 0, 1024)])
def test_one_round_decode_attention_gives_the_bits_of_the_persistent_kernel(dev, status, nq, nkv, d, page, window, segment):
    """With few tokens the decode attention runs as one CTA per (token, kv head, segment), the
    segments of a token in a thread-block cluster that merges them through the first CTA's shared
    memory; with many it walks over its items and merges through global memory. At the same segment
    length both give the same bits, in the plain form and in the fused one, whatever the lengths
    (one key, one segment, a window that hides the first segments); and the rule takes the
    kernel with one CTA per item exactly where it says."""
    from vosti_b200 import ops
    lib = ops.library()
    # few enough tokens for all CTAs to run at once: clusters of more than 8 CTAs only serve up to 8 (token, kv head)
    # pairs, and with head size 256 an SM holds one CTA, so that fewer clusters fit the GPU at once
    lengths = [2047, 300, 1, 1500, 17, 1024, 33, 640, 2000, 129, 64, 65, 1999, 5, 1025, 511]
    lens_k = lengths[: max(1, (8 if -(-2047 // segment) > 8 or d > 128 else 16) // nkv)]
    lens_q = [1] * len(lens_k)
    case = paged_case(dev, torch.bfloat16, lens_q, lens_k, nq, nkv, d, page)
    scale = d ** -0.5
    out = {}
    ops.set_decode_segment(segment)
    try:
        for once in (True, False):
            ops.set_decode_once(once)
            out[once] = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, scale, window, "decode")
            assert lib.vosti_attention_decode_last_kernel() == (2 if once else 1)
        assert torch.equal(out[True], out[False])
        want = reference_attention(case, scale, window)
        assert torch.allclose(out[True].float().cpu(), want, atol=2e-2, rtol=2e-2)
        # the fused form: the same partial sums through both kernels
        B, heads, splits = len(lens_k), nq + 2 * nkv, 6
        gen = torch.Generator(device=dev).manual_seed(d + nq)
        partial = torch.randn(splits, B, heads * d, device=dev, generator=gen) * 0.6
        qw = (1 + 0.1 * torch.randn(d, device=dev, generator=gen)).bfloat16()
        kw = (1 + 0.1 * torch.randn(d, device=dev, generator=gen)).bfloat16()
        cos, sin = (t.to(dev).contiguous() for t in plain.rope_tables(torch.arange(2100), d, 1e4))
        table, positions = case["table"].to(dev), case["positions"].to(dev)
        slots = torch.tensor([int(table[b, (n - 1) // page]) * page + (n - 1) % page for b, n in enumerate(lens_k)],
                             dtype=torch.int32, device=dev)
        fused, caches = {}, {}
        for once in (True, False):
            ops.set_decode_once(once)
            k, v = dev_cache(case, "k_cache", dev, torch.bfloat16).clone(), dev_cache(case, "v_cache", dev, torch.bfloat16).clone()
            k, v = torch.nan_to_num(k), torch.nan_to_num(v)
            fused[once] = ops.attention_decode_fused(
                ops.PartialSum(partial, splits, B, heads * d, torch.bfloat16, status), k, v, positions=positions,
                request_of=case["request_of"].to(dev), block_table=table, slot_mapping=slots, page_size=page, nq=nq, nkv=nkv,
                head_dim=d, max_kv_len=max(lens_k), scale=scale, window=window, q_norm_w=qw, k_norm_w=kw, eps=1e-6, cos=cos,
                sin=sin, status=status)
            caches[once] = (k, v)
            assert lib.vosti_attention_decode_last_kernel() == (2 if once else 1)
        assert torch.equal(fused[True], fused[False]) and torch.isfinite(fused[True]).all()
        assert torch.equal(caches[True][0], caches[False][0]) and torch.equal(caches[True][1], caches[False][1])
        assert status.item() == 0
    finally:
        ops.set_decode_once(True)
        ops.set_decode_segment(0)


def test_decode_attention_kernels_by_launch_shape(dev, status):
    """Pages of no multiple of 16 tokens, or a context too long for 8 segments of 4096 keys: the
    persistent kernel runs. More (token, kv head) pairs than CTAs fit the GPU at once: the kernel
    with one CTA per item still runs, in waves. The results are right either way."""
    from vosti_b200 import ops
    lib = ops.library()
    nq, nkv, d = 8, 2, 64
    for page, lens_k, kernel in ((16, [200] * 400, 2), (8, [300, 17, 64], 1), (16, [33000, 5, 70, 1, 900], 1)):
        lens_q = [1] * len(lens_k)
        case = paged_case(dev, torch.bfloat16, lens_q, lens_k, nq, nkv, d, page)
        out = _run_tc_attention(dev, status, case, lens_q, lens_k, nq, nkv, d, page, d ** -0.5, 0, "decode")
        assert lib.vosti_attention_decode_last_kernel() == kernel, (page, len(lens_k))
        want = reference_attention(case, d ** -0.5, 0)
        assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    assert status.item() == 0

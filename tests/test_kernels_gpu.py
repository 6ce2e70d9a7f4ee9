"""Each kernel alone against a plain PyTorch restatement of the same operation, at sizes
other than the tiny models': head sizes in steps of 16, head counts and groups that are
no power of two, odd widths and vocabularies."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def ops():
    from rust_mlx_b200.kernels import ops as o
    return o


def rnd(shape, dtype, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, width, vocab", [(1, 16, 3), (37, 200, 509), (300, 4096, 1000)])
def test_embedding(dtype, n, width, vocab):
    table = rnd((vocab, width), DT[dtype])
    ids = torch.randint(0, vocab, (n,), dtype=torch.int32, device=DEV)
    h = torch.empty(n, width, dtype=torch.float32, device=DEV)
    ops().embedding(ids, table, h)
    assert torch.equal(h, table[ids.long()].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, width, ld", [(1, 16, 16), (7, 99, 99), (33, 1000, 1536), (300, 6144, 6144)])
def test_add_bias(dtype, n, width, ld):
    """x[t, :] += bias with one rounding, also on some columns of wider rows (the rest untouched)."""
    dt = DT[dtype]
    full = rnd((n, ld), dt, 1.0, 3)
    bias = rnd((width,), torch.float32, 0.5, 4)
    before = full.clone()
    ops().add_bias(full[:, :width], bias)
    want = (before[:, :width].float() + bias).to(dt)
    assert torch.equal(full[:, :width], want)
    assert torch.equal(full[:, width:], before[:, width:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, width", [(1, 16), (5, 96), (33, 1000), (64, 4096), (3, 12288 + 8)])
def test_add_rmsnorm(dtype, n, width):
    dt = DT[dtype]
    h = rnd((n, width), torch.float32, 2.0, 1)
    delta = rnd((n, width), dt, 0.5, 2)
    w = (1 + 0.1 * torch.randn(width)).to(DEV)
    eps = 1e-5
    x = torch.empty(n, width, dtype=dt, device=DEV)
    h0 = h.clone()
    ops().add_rmsnorm(h, delta, w, eps, x)
    v = h0.double() + delta.double()
    want = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.double()
    assert torch.allclose(h, v.float(), atol=1e-6)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert (x.double() - want).abs().max().item() < tol * max(1.0, want.abs().max().item())
    # without a delta, and for chosen rows only (h untouched)
    rows = torch.tensor([n - 1, 0], dtype=torch.int32, device=DEV)
    x2 = torch.empty(2, width, dtype=dt, device=DEV)
    h1 = h.clone()
    ops().add_rmsnorm(h, None, w, eps, x2, rows=rows)
    assert torch.equal(h, h1)
    v = h1.double()[rows.long()]
    want = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.double()
    assert (x2.double() - want).abs().max().item() < tol * max(1.0, want.abs().max().item())


def test_rmsnorm_rows_do_not_depend_on_the_batch():
    h = rnd((40, 777), torch.float32, 1.0, 3)
    w = torch.ones(777, device=DEV)
    a = torch.empty(40, 777, device=DEV)
    b = torch.empty(1, 777, device=DEV)
    ops().add_rmsnorm(h.clone(), None, w, 1e-6, a)
    ops().add_rmsnorm(h[17:18].clone(), None, w, 1e-6, b)
    assert torch.equal(a[17], b[0])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, inter", [(1, 16), (7, 160), (130, 1111)])
def test_swiglu(dtype, n, inter):
    dt = DT[dtype]
    gu = rnd((n, 2 * inter), dt, 3.0)
    out = torch.empty(n, inter, dtype=dt, device=DEV)
    ops().swiglu(gu, out)
    g, u = gu.double()[:, :inter], gu.double()[:, inter:]
    want = g * torch.sigmoid(g) * u
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, inter, block", [(3, 128, 64), (70, 192, 64), (5, 24, 8), (9, 30, 6)])
def test_swiglu_over_blocks_of_gate_and_up(dtype, n, inter, block):
    dt = DT[dtype]
    gu = rnd((n, 2 * inter), dt, 3.0, 4)
    out = torch.empty(n, inter, dtype=dt, device=DEV)
    ops().swiglu(gu, out, block)
    v = gu.double().reshape(n, inter // block, 2, block)
    g, u = v[:, :, 0].reshape(n, inter), v[:, :, 1].reshape(n, inter)
    want = g * torch.sigmoid(g) * u
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.parametrize("m, n, k", [(1, 16, 16), (3, 509, 96), (70, 130, 257), (128, 64, 4096), (200, 1000, 33)])
def test_gemm_plain_float32(m, n, k):
    a, w = rnd((m, k), torch.float32, 1.0, 1), rnd((n, k), torch.float32, 1.0, 2)
    out = torch.empty(m, n, device=DEV)
    ops().gemm_plain(a, w, out)
    want = a.double() @ w.double().t()
    assert (out.double() - want).abs().max().item() < 1e-5 * math.sqrt(k) * 4
    # a row's result does not depend on the other rows
    one = torch.empty(1, n, device=DEV)
    ops().gemm_plain(a[m // 2:m // 2 + 1].contiguous(), w, one)
    assert torch.equal(one[0], out[m // 2])


@pytest.mark.parametrize("m, n, k", [(1, 48, 64), (5, 509, 96), (130, 200, 1000)])
def test_gemm_plain_bfloat16_and_float_logits(m, n, k):
    a, w = rnd((m, k), torch.bfloat16, 1.0, 1), rnd((n, k), torch.bfloat16, 1.0, 2)
    want = a.double() @ w.double().t()
    out32 = torch.empty(m, n, device=DEV)
    ops().gemm_plain(a, w, out32)
    assert (out32.double() - want).abs().max().item() < 1e-4 * math.sqrt(k)
    out16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops().gemm_plain(a, w, out16)
    assert ((out16.double() - want).abs() <= 1e-2 * (1 + want.abs())).all()


@pytest.mark.parametrize("m, n, k", [(1, 48, 64), (8, 6144, 4096), (64, 509 * 2, 96), (300, 200, 1000)])
def test_linear_bfloat16(m, n, k):
    a, w = rnd((m, k), torch.bfloat16, 1.0, 1), rnd((n, k), torch.bfloat16, 0.05, 2)
    want = a.double() @ w.double().t()
    for odt in (torch.bfloat16, torch.float32):
        out = torch.empty(m, n, dtype=odt, device=DEV)
        ops().linear(a, w, out)
        tol = 1e-2 if odt == torch.bfloat16 else 2e-3
        assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()


def paged_setup(lengths, nkv, hd, page, dtype, seed=0, extra_pages=3):
    """Random K, V for sequences of the given lengths scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lengths) + extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    k_pool = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype)
    v_pool = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype)
    max_entries = max(-(-n // page) for n in lengths)
    table = torch.full((len(lengths), max_entries), -1, dtype=torch.int32)
    ks, vs = [], []
    for s, n in enumerate(lengths):
        k = torch.randn(n, nkv, hd, generator=g).to(dtype)
        v = torch.randn(n, nkv, hd, generator=g).to(dtype)
        ks.append(k)
        vs.append(v)
        for i in range(-(-n // page)):
            p = perm.pop()
            table[s, i] = p
            rows = k[i * page:(i + 1) * page]
            k_pool[p, :, :rows.shape[0]] = rows.transpose(0, 1)
            v_pool[p, :, :rows.shape[0]] = v[i * page:(i + 1) * page].transpose(0, 1)
    return k_pool.to(DEV), v_pool.to(DEV), table.to(DEV), ks, vs


def plain_attention(q, k, v, qpos, window, scale):
    """q: [T, nq, hd] at positions qpos; k, v: [S, nkv, hd] for positions 0..S-1."""
    T, nq, hd = q.shape
    group = nq // k.shape[1]
    kpos = torch.arange(k.shape[0])
    allowed = kpos[None, :] <= qpos[:, None]
    if window:
        allowed &= kpos[None, :] > qpos[:, None] - window
    out = torch.empty(T, nq, hd, dtype=torch.float64)
    for h in range(nq):
        s = (q[:, h].double() @ k[:, h // group].double().t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, h // group].double()
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, hd, page, window", [
    (4, 2, 16, 16, 0), (6, 2, 32, 8, 20), (5, 5, 48, 4, 0), (12, 4, 80, 32, 37), (32, 8, 128, 64, 0),
    (3, 1, 256, 16, 0), (7, 1, 112, 2, 5)])
def test_attention_plain_over_pages(dtype, nq, nkv, hd, page, window):
    """Portions of several sequences and single decoded tokens in one batch; NaN in every
    slot of the pool that must not be read."""
    dt = DT[dtype]
    lengths = [70, 1, 33, 130]
    new = [9, 1, 33, 1]                    # the last `new` tokens of each sequence are this step's queries
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, dt, seed=hd)
    qs, pos, sidx = [], [], []
    for s, (n, c) in enumerate(zip(lengths, new)):
        qs.append(torch.randn(c, nq, hd).to(dt))
        pos += list(range(n - c, n))
        sidx += [s] * c
    q = torch.cat(qs).to(DEV)
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    seq_index = torch.tensor(sidx, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = hd ** -0.5
    ops().attention_plain(q.reshape(-1, nq * hd), k_pool, v_pool, positions, seq_index, table, page, out.reshape(-1, nq * hd),
                          nq, nkv, hd, window, scale, status)
    assert status.item() == 0
    at = 0
    tol = 2e-5 if dtype == "float32" else 1e-2
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, scale)
        got = out[at:at + c].double().cpu()
        assert not torch.isnan(got).any()
        assert (got - want).abs().max().item() < tol
        at += c


def test_attention_finds_a_far_key_among_hundreds():
    """One key far back matches the query strongly: the output must be that key's value.
    With random keys a kernel that skips or misplaces it would still pass a tolerance."""
    nq, nkv, hd, page = 4, 2, 32, 8
    n = 700
    k_pool, v_pool, table, ks, vs = paged_setup([n], nkv, hd, page, torch.float32, seed=5)
    for target in (0, 7, 8, 255, 256, 511, n - 1):
        q = torch.randn(1, nq, hd) * 0.1
        k = ks[0].clone()
        k[target] = 0
        k[target, :, 3] = 40.0
        q[0, :, 3] = 40.0
        pg, slot = table[0, target // page].item(), target % page
        k_pool[pg, :, slot] = k[target].to(DEV)
        out = torch.empty(1, nq * hd, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().attention_plain(q.reshape(1, -1).to(DEV), k_pool, v_pool, torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                              torch.zeros(1, dtype=torch.int32, device=DEV), table, page, out, nq, nkv, hd, 0, hd ** -0.5, status)
        want = vs[0][target].repeat_interleave(nq // nkv, 0).reshape(-1)
        assert (out[0].cpu() - want).abs().max().item() < 1e-4, target
        k_pool[pg, :, slot] = ks[0][target].to(DEV)


def test_attention_window_edge():
    """The key just outside the window carries a huge score: it must not be seen; the key
    just inside must."""
    nq, nkv, hd, page, window, n = 2, 1, 16, 4, 10, 50
    k_pool, v_pool, table, ks, vs = paged_setup([n], nkv, hd, page, torch.float32, seed=6)
    q = torch.zeros(1, nq, hd)
    q[0, :, 0] = 30.0
    for target, seen in ((n - window - 1, False), (n - window, True)):
        kp = k_pool.clone()
        kp[table[0, target // page].item(), :, target % page, 0] = 30.0
        out = torch.empty(1, nq * hd, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().attention_plain(q.reshape(1, -1).to(DEV), kp, v_pool, torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                              torch.zeros(1, dtype=torch.int32, device=DEV), table, page, out, nq, nkv, hd, window, hd ** -0.5, status)
        hit = (out[0, :hd].cpu() - vs[0][target, 0]).abs().max().item() < 1e-3
        assert hit == seen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, hd, rot, page, norm", [
    (4, 2, 16, 16, 16, True), (6, 2, 32, 32, 8, True), (5, 5, 48, 24, 4, False), (32, 8, 128, 128, 64, True),
    (3, 1, 80, 0, 2, True)])
def test_qk_norm_rotation_and_cache_write(dtype, nq, nkv, hd, rot, page, norm):
    dt = DT[dtype]
    lengths, new = [21, 6, 40], [5, 6, 1]
    n_tok = sum(new)
    n_pages = sum(-(-n // page) for n in lengths) + 2
    table = torch.full((3, max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages).tolist()
    for s, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[s, i] = perm.pop()
    pos, sidx = [], []
    for s, (n, c) in enumerate(zip(lengths, new)):
        pos += list(range(n - c, n))
        sidx += [s] * c
    qkv = rnd((n_tok, (nq + 2 * nkv) * hd), dt, 1.0, 3)
    qn = (1 + 0.2 * torch.randn(hd)).to(DEV) if norm else None
    kn = (1 + 0.2 * torch.randn(hd)).to(DEV) if norm else None
    theta, eps = 10000.0, 1e-5
    inv_freq = (theta ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))).float().to(DEV) if rot else None
    k_pool = torch.zeros(n_pages, nkv, page, hd, dtype=dt, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty(n_tok, nq * hd, dtype=dt, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    table_dev = table.to(DEV)
    ops().qk_rope_cache(qkv, qn, kn, eps, inv_freq, rot, positions, torch.tensor(sidx, dtype=torch.int32, device=DEV),
                        table_dev, page, k_pool, v_pool, q_out, nq, nkv, hd, True, status)
    assert status.item() == 0
    x = qkv.double().cpu()
    q = x[:, :nq * hd].reshape(n_tok, nq, hd)
    k = x[:, nq * hd:(nq + nkv) * hd].reshape(n_tok, nkv, hd)
    v = x[:, (nq + nkv) * hd:].reshape(n_tok, nkv, hd)

    def normed(t, w):
        if w is None:
            return t
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.double().cpu()

    def rotate(t):
        if rot == 0:
            return t
        half = rot // 2
        ang = (positions.cpu().float()[:, None] * inv_freq.cpu()[None, :]).double()[:, None, :]
        a, b = t[..., :half], t[..., half:rot]
        out = t.clone()
        out[..., :half] = a * ang.cos() - b * ang.sin()
        out[..., half:rot] = b * ang.cos() + a * ang.sin()
        return out

    tol = 1e-5 if dtype == "float32" else 3e-2
    want_q = rotate(normed(q, qn))
    assert (q_out.double().cpu().reshape(n_tok, nq, hd) - want_q).abs().max().item() < tol
    if rot:
        # the same with the step's cosines and sines formed once (for head 128 in bfloat16 a kernel of its own)
        angles = torch.empty(n_tok, rot, device=DEV)
        ops().rope_table(positions, inv_freq, rot, angles)
        ang = positions.cpu().float()[:, None] * inv_freq.cpu()[None, :]
        assert torch.allclose(angles.cpu(), torch.cat([ang.cos(), ang.sin()], 1), atol=1e-6)
        q2, k2, v2 = torch.empty_like(q_out), torch.zeros_like(k_pool), torch.zeros_like(v_pool)
        ops().qk_rope_cache(qkv, qn, kn, eps, inv_freq, rot, positions, torch.tensor(sidx, dtype=torch.int32, device=DEV),
                            table_dev, page, k2, v2, q2, nq, nkv, hd, True, status, cos_sin=angles)
        assert (q2.double() - q_out.double()).abs().max().item() <= (0 if not (dtype == "bfloat16" and hd == 128) else 3e-2)
        assert (k2.double() - k_pool.double()).abs().max().item() <= (0 if not (dtype == "bfloat16" and hd == 128) else 3e-2)
        assert torch.equal(v2, v_pool) and status.item() == 0
    want_k = rotate(normed(k, kn))
    for t in range(n_tok):
        pg, slot = table[sidx[t], pos[t] // page].item(), pos[t] % page
        assert (k_pool[pg, :, slot].double().cpu() - want_k[t]).abs().max().item() < tol
        assert torch.equal(v_pool[pg, :, slot].cpu(), qkv[t, (nq + nkv) * hd:].reshape(nkv, hd).cpu())
    # nothing else was written
    written = {(table[sidx[t], pos[t] // page].item(), pos[t] % page) for t in range(n_tok)}
    mask = torch.ones(n_pages, page, dtype=torch.bool)
    for pg, slot in written:
        mask[pg, slot] = False
    assert k_pool.cpu().transpose(1, 2)[mask].abs().max().item() == 0


def test_cache_write_without_a_page_is_reported_not_done():
    nq, nkv, hd, page = 2, 1, 16, 4
    qkv = rnd((1, 4 * hd), torch.float32)
    table = torch.full((1, 2), -1, dtype=torch.int32, device=DEV)
    k_pool = torch.zeros(2, nkv, page, hd, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().qk_rope_cache(qkv, None, None, 0.0, None, 0, torch.tensor([5], dtype=torch.int32, device=DEV),
                        torch.zeros(1, dtype=torch.int32, device=DEV), table, page, k_pool, v_pool,
                        torch.empty(1, nq * hd, device=DEV), nq, nkv, hd, True, status)
    assert status.item() == 1 and k_pool.abs().max().item() == 0


@pytest.mark.parametrize("vocab", [3, 509, 151936])
def test_greedy_takes_the_lowest_id_on_ties(vocab):
    logits = torch.randn(5, vocab, device=DEV)
    top = logits.max().item() + 1
    logits[1, vocab - 1] = top
    logits[1, vocab // 2] = top
    logits[2, 0] = top
    logits[3, :] = 0.25
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops().sample(logits, None, None, out)
    want = [int(torch.nonzero(r == r.max())[0, 0]) for r in logits.cpu()]
    assert out.tolist() == want and want[1] == vocab // 2 and want[3] == 0


@pytest.mark.parametrize("vocab", [7, 509, 50000])
def test_temperature_sampling_inverts_the_cumulative_sum(vocab):
    torch.manual_seed(0)
    logits = (torch.randn(64, vocab) * 3).to(DEV)
    temps = torch.full((64,), 0.8, device=DEV)
    temps[::7] = 0.0
    u = torch.rand(64, device=DEV)
    out = torch.empty(64, dtype=torch.int32, device=DEV)
    ops().sample(logits, temps, u, out)
    p = torch.softmax(logits.double().cpu() / 0.8, -1)
    cdf = torch.cumsum(p, -1)
    for r, t in enumerate(out.tolist()):
        if r % 7 == 0:
            assert t == int(logits[r].argmax())
            continue
        lo = cdf[r, t - 1].item() if t > 0 else 0.0
        assert lo - 1e-5 <= u[r].item() <= cdf[r, t].item() + 1e-5
    # rows do not depend on the batch
    one = torch.empty(1, dtype=torch.int32, device=DEV)
    ops().sample(logits[5:6], temps[5:6], u[5:6], one)
    assert one.item() == out[5].item()
    # frequencies follow the distribution
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device=DEV).repeat(4000, 1)
    draws = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops().sample(small, torch.ones(4000, device=DEV), torch.rand(4000, device=DEV), draws)
    freq = torch.bincount(draws.long().cpu(), minlength=4).double() / 4000
    assert (freq - torch.softmax(small[0].double().cpu(), -1)).abs().max().item() < 0.03


def test_kernels_refuse_what_they_cannot_do():
    from rust_mlx_b200.kernels.library import KernelError
    o = ops()
    with pytest.raises(KernelError, match="CUDA device"):
        o.swiglu(torch.zeros(2, 8), torch.zeros(2, 4))
    with pytest.raises(KernelError, match="dtype"):
        o.swiglu(torch.zeros(2, 8, dtype=torch.float16, device=DEV), torch.zeros(2, 4, dtype=torch.float16, device=DEV))
    q = torch.zeros(1, 66 * 16, device=DEV)
    pool = torch.zeros(1, 1, 4, 16, device=DEV)
    i32 = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="32 query heads"):
        o.attention_plain(q, pool, pool, i32, i32, i32.view(1, 1), 4, q.clone(), 66, 1, 16, 0, 1.0, i32)
    with pytest.raises(KernelError, match="rotary_dim"):
        o.qk_rope_cache(torch.zeros(1, 48, device=DEV), None, None, 0.0, torch.zeros(8, device=DEV), 18, i32, i32,
                        i32.view(1, 1), 4, pool, pool, torch.zeros(1, 16, device=DEV), 1, 1, 16, True, i32)


class _Batch:
    """The few fields of a step's batch that the attention wrappers read."""

    def __init__(self, lengths, new, status):
        starts = [0]
        for c in new:
            starts.append(starts[-1] + c)
        self.q_start_host, self.n_seqs, self.max_seq_len, self.max_q_len = starts, len(lengths), max(lengths), max(new)
        self.q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        pos, sidx = [], []
        for s, (n, c) in enumerate(zip(lengths, new)):
            pos += list(range(n - c, n))
            sidx += [s] * c
        self.positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
        self.seq_index = torch.tensor(sidx, dtype=torch.int32, device=DEV)
        self.status = status


@pytest.mark.parametrize("splits", [None, 1, 3])
@pytest.mark.parametrize("nq, nkv, hd, page, window", [
    (4, 2, 16, 16, 0), (6, 2, 32, 8, 20), (5, 5, 64, 4, 0), (12, 4, 96, 32, 37), (32, 8, 128, 64, 0),
    (16, 1, 128, 16, 0), (7, 7, 128, 2, 5), (8, 2, 64, 64, 100)])
def test_attention_flash_over_pages(nq, nkv, hd, page, window, splits):
    """Portions of several sequences (longer than one query tile, crossing key tiles) beside
    single decoded tokens; NaN in every slot of the pool that must not be read.  Outputs are
    bfloat16: the bound is 1e-2 * (1 + |value|), half a last bit at the largest values."""
    from rust_mlx_b200.engine.workspace import Workspace
    torch.manual_seed(nq * 1000 + hd)
    lengths = [200, 1, 33, 130, 300, 64]
    new = [70, 1, 33, 1, 1, 64]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=hd + nq)
    qs = [torch.randn(c, nq, hd).to(torch.bfloat16) for c in new]
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    out = torch.full_like(q, float("nan"))
    scale = hd ** -0.5
    ops().attention_flash(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, window, scale, Workspace(DEV), n_splits=splits)
    assert status.item() == 0
    at = 0
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, scale)
        got = out[at:at + c].double().cpu().reshape(c, nq, hd)
        assert not torch.isnan(got).any()
        assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (s, n, c)
        at += c


@pytest.mark.parametrize("splits", [1, 5])
def test_attention_flash_finds_a_far_key_and_respects_the_window_edge(splits):
    from rust_mlx_b200.engine.workspace import Workspace
    nq, nkv, hd, page, n = 8, 2, 64, 16, 900
    k_pool, v_pool, table, ks, vs = paged_setup([n], nkv, hd, page, torch.bfloat16, seed=8)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch([n], [1], status)
    ws = Workspace(DEV)
    for window, target, seen in ((0, 0, True), (0, 63, True), (0, 64, True), (0, 511, True), (0, n - 1, True),
                                 (100, n - 101, False), (100, n - 100, True)):
        q = torch.zeros(1, nq, hd)
        q[0, :, 5] = 24.0
        kp = k_pool.clone()
        kp[table[0, target // page].item(), :, target % page, :] = 0
        kp[table[0, target // page].item(), :, target % page, 5] = 24.0
        out = torch.empty(1, nq * hd, dtype=torch.bfloat16, device=DEV)
        ops().attention_flash(q.reshape(1, -1).to(torch.bfloat16).to(DEV), kp, v_pool, batch, table, page, out, nq, nkv, hd,
                              window, hd ** -0.5, ws, n_splits=splits)
        want = vs[0][target].float().repeat_interleave(nq // nkv, 0).reshape(-1)
        hit = (out[0].float().cpu() - want).abs().max().item() < 2e-2
        assert hit == seen, (window, target)


def test_attention_flash_rows_do_not_depend_on_the_batch():
    """The same token alone and inside a larger batch gives the same bits (one split)."""
    from rust_mlx_b200.engine.workspace import Workspace
    nq, nkv, hd, page = 8, 2, 128, 16
    lengths, new = [150, 90], [40, 1]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=2)
    qs = [torch.randn(c, nq, hd).to(torch.bfloat16) for c in new]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ws = Workspace(DEV)
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    out = torch.empty_like(q)
    ops().attention_flash(q, k_pool, v_pool, _Batch(lengths, new, status), table, page, out, nq, nkv, hd, 0, hd ** -0.5, ws, n_splits=1)
    # the last 7 tokens of sequence 0 as a portion of their own (the same arrangement of warps)
    q2 = qs[0][-7:].to(DEV).reshape(-1, nq * hd)
    out2 = torch.empty_like(q2)
    ops().attention_flash(q2, k_pool, v_pool, _Batch([150], [7], status), table[:1], page, out2, nq, nkv, hd, 0, hd ** -0.5, ws, n_splits=1)
    assert torch.equal(out2, out[33:40])


@pytest.mark.parametrize("splits", [None, 1, 4, 7, 12])   # 2..8: merged inside a cluster; more: through global memory
@pytest.mark.parametrize("nq, nkv, hd, page, window, new_len", [
    (4, 2, 16, 16, 0, 1), (6, 2, 32, 8, 20, 1), (32, 8, 128, 64, 0, 1), (16, 1, 128, 16, 0, 1), (8, 2, 64, 4, 50, 4),
    (5, 5, 96, 2, 0, 16), (64, 8, 128, 64, 0, 2), (6, 3, 64, 8, 70, 3), (12, 4, 128, 32, 33, 1), (4, 4, 64, 128, 0, 2),
    (40, 8, 128, 16, 0, 1)])
def test_attention_flash_decoding_arrangement(nq, nkv, hd, page, window, new_len, splits):
    """Every sequence brings so few tokens that a tile has at most 16 rows: the kernel then
    spreads a tile's keys over its warps and combines them."""
    from rust_mlx_b200.engine.workspace import Workspace
    torch.manual_seed(nq * 1000 + hd + new_len)
    lengths = [200, 17, 33, 130, 700, 64, 65, 16]
    new = [new_len] * len(lengths)
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=hd + nq)
    qs = [torch.randn(c, nq, hd).to(torch.bfloat16) for c in new]
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    out = torch.full_like(q, float("nan"))
    ops().attention_flash(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, window, hd ** -0.5, Workspace(DEV), n_splits=splits)
    assert status.item() == 0
    at = 0
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, hd ** -0.5)
        got = out[at:at + c].double().cpu().reshape(c, nq, hd)
        assert not torch.isnan(got).any()
        assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (s, n, c)
        at += c


@pytest.mark.parametrize("hd, window", [(128, 0), (64, 0), (128, 30000)])
def test_decoding_attention_over_a_very_long_context(hd, window):
    """One decoded token of one request against 70,000 keys: the rule then splits the keys more than eight
    ways (no cluster is that large: the shares go through global memory and the last block adds them), and
    the block table (more than a thousand pages) is longer than what a block keeps of it in shared memory.
    A needle far back: one key that the query is scaled to find."""
    from rust_mlx_b200.engine.workspace import Workspace
    nq, nkv, page, n = 8, 2, 64, 70000
    assert ops().flash_splits(1, nkv, n) > 8
    k_pool, v_pool, table, ks, vs = paged_setup([n, 40], nkv, hd, page, torch.bfloat16, seed=hd)
    torch.manual_seed(1)
    needle = 41234
    qs = [torch.randn(1, nq, hd).to(torch.bfloat16), torch.randn(1, nq, hd).to(torch.bfloat16)]
    qs[0][0, :, 7] = 30.0
    k_pool[table[0, needle // page].item(), :, needle % page, :] = 0
    k_pool[table[0, needle // page].item(), :, needle % page, 7] = 30.0
    ks[0][needle] = 0
    ks[0][needle, :, 7] = 30.0
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for lengths, new, which in (([n], [1], [0]), ([n, 40], [1, 1], [0, 1])):
        q = torch.cat([qs[i] for i in which]).to(DEV).reshape(-1, nq * hd)
        out = torch.full_like(q, float("nan"))
        ops().attention_flash(q, k_pool, v_pool, _Batch(lengths, new, status), table[:len(lengths)], page, out, nq, nkv, hd, window,
                              hd ** -0.5, Workspace(DEV))
        assert status.item() == 0
        for row, i in enumerate(which):
            want = plain_attention(qs[i], ks[i], vs[i], torch.tensor([lengths[row] - 1]), window, hd ** -0.5)
            got = out[row].double().cpu().reshape(1, nq, hd)
            assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (lengths, i, (got - want).abs().max().item())
        if window == 0:   # the needle was found: the first request's output is its value
            assert (out[0].float().cpu().reshape(nq, hd) - vs[0][needle].float().repeat_interleave(nq // nkv, 0)).abs().max() < 3e-2


@pytest.mark.parametrize("m, n, k, splits", [
    (1, 128, 64, 1), (16, 128, 128, 1), (1, 6144, 4096, None), (8, 4096, 4096, 4), (8, 24576, 4096, None),
    (3, 509, 96, 1), (17, 1000, 136, 2), (33, 4096, 12288, None), (64, 2048, 4096, 1), (64, 1100, 520, 3),
    (5, 130, 8, 1), (40, 96, 264, 1)])
def test_gemm_tcgen05(m, n, k, splits):
    """The tcgen05/TMA product for few rows: sizes that are no multiple of the 128-row tile
    or the 64-wide k block, with and without split-K, bfloat16 and float results."""
    a, w = rnd((m, k), torch.bfloat16, 1.0, 1), rnd((n, k), torch.bfloat16, 0.05, 2)
    want = a.double() @ w.double().t()
    for odt in (torch.float32, torch.bfloat16):
        out = torch.full((m, n), float("nan"), dtype=odt, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().gemm_tcgen05(a, w, out, status=status, splits=splits)
        assert status.item() == 0
        tol = 1e-2 if odt == torch.bfloat16 else 1e-4
        assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()
    # split-K leaves its counters at zero: a second call gives the same bits
    out2 = torch.empty_like(out)
    ops().gemm_tcgen05(a, w, out2, status=status, splits=splits)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("m, inter, k, splits", [(1, 64, 64, 1), (8, 12288, 4096, None), (20, 192, 520, 2), (64, 1024, 4096, 1),
                                                  (33, 640, 1032, 4)])
def test_gemm_tcgen05_with_swiglu_epilogue(m, inter, k, splits):
    """Weights in blocks of 64 gate rows and their 64 up rows: the product's epilogue gives
    silu(gate) * up, [m, inter], in float and rounded once."""
    a = rnd((m, k), torch.bfloat16, 1.0, 1)
    gate, up = rnd((inter, k), torch.bfloat16, 0.05, 2), rnd((inter, k), torch.bfloat16, 0.05, 3)
    w = torch.stack([gate.view(inter // 64, 64, k), up.view(inter // 64, 64, k)], dim=1).reshape(2 * inter, k).contiguous()
    g, u = a.double() @ gate.double().t(), a.double() @ up.double().t()
    want = g * torch.sigmoid(g) * u
    for cluster in (True, False):
        for odt in (torch.bfloat16, torch.float32):
            out = torch.full((m, inter), float("nan"), dtype=odt, device=DEV)
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            ops().gemm_tcgen05(a, w, out, status=status, splits=splits, cluster=cluster, swiglu=True)
            assert status.item() == 0
            tol = 1e-2 if odt == torch.bfloat16 else 2e-4
            assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()


def test_gemm_tcgen05_rows_do_not_depend_on_the_batch():
    a, w = rnd((8, 4096), torch.bfloat16, 1.0, 1), rnd((1024, 4096), torch.bfloat16, 0.05, 2)
    out8 = torch.empty(8, 1024, device=DEV)
    out1 = torch.empty(1, 1024, device=DEV)
    ops().gemm_tcgen05(a, w, out8, splits=2)
    ops().gemm_tcgen05(a[3:4].contiguous(), w, out1, splits=2)
    assert torch.equal(out8[3], out1[0])


def test_gemm_tcgen05_refuses_what_it_cannot_do():
    from rust_mlx_b200.kernels.library import KernelError
    a, w = rnd((65, 64), torch.bfloat16), rnd((128, 64), torch.bfloat16)
    with pytest.raises(KernelError, match="1..64 rows"):
        ops().gemm_tcgen05(a, w, torch.empty(65, 128, dtype=torch.bfloat16, device=DEV))
    a, w = rnd((4, 60), torch.bfloat16), rnd((128, 60), torch.bfloat16)
    with pytest.raises(KernelError, match="K % 8"):
        ops().gemm_tcgen05(a, w, torch.empty(4, 128, dtype=torch.bfloat16, device=DEV))
    assert not ops().prefers_tcgen05(4, 128, 60)


@pytest.mark.parametrize("nq, nkv, page, window", [(32, 8, 64, 0), (8, 8, 16, 0), (16, 1, 8, 0), (4, 2, 32, 50), (8, 2, 128, 0),
                                                   (32, 8, 64, 300)])
@pytest.mark.parametrize("per_block, runs", [(1, 1), (2, 1), (2, 3), (1, 2)])
@pytest.mark.parametrize("hd", [128, 64])
def test_attention_tcgen05_over_pages(nq, nkv, page, window, per_block, runs, hd):
    """Prompt portions on the tcgen05 tensor cores (head sizes 128 and 64): several sequences whose portions span
    more than one tile of 128 rows and several key tiles, beside short ones; NaN in every slot of the pool
    that must not be read.  With two query tiles a block (they share the key tiles) and with one; with every
    tile's keys in one run and in several (some of which are empty for short sequences)."""
    torch.manual_seed(nq * 100 + page)
    lengths = [300, 40, 33, 130, 700, 64, 1]
    new = [170, 40, 5, 130, 260, 64, 1]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=page + nq)
    qs = [torch.randn(c, nq, hd).to(torch.bfloat16) for c in new]
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    out = torch.full_like(q, float("nan"))
    scale = hd ** -0.5
    ops().attention_tcgen05(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, window, scale, per_block=per_block, n_splits=runs)
    assert status.item() == 0
    at = 0
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, scale)
        got = out[at:at + c].double().cpu().reshape(c, nq, hd)
        assert not torch.isnan(got).any(), (s, n, c)
        assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (s, n, c, (got - want).abs().max().item())
        at += c


@pytest.mark.parametrize("nq, nkv, hd", [(6, 2, 64), (8, 2, 64), (6, 2, 128), (8, 2, 128), (6, 2, 32), (4, 2, 96), (4, 4, 16)])
@pytest.mark.parametrize("lengths, new", [([644, 1], [196, 1]), ([1, 644], [1, 196]), ([39, 39, 288], [1, 1, 12]),
                                          ([288, 39, 39], [12, 1, 1]), ([700, 50], [196, 2]), ([298, 63, 5], [150, 1, 5])])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_of_a_mixed_step_in_two_launches(nq, nkv, hd, lengths, new, window):
    """``ops.attention`` gives the decoded tokens of a mixed step to the key-split kernel and the portions to
    the kernel for portions, each launch with a run of the step's sequences; q, the output and the partial sums
    of split keys are the whole step's.  Long contexts, so that keys are split and the shares have to be added
    for the launch's own rows only (the other rows belong to the other launch)."""
    from rust_mlx_b200.engine.workspace import Workspace
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, 32, torch.bfloat16, seed=hd + nq)
    torch.manual_seed(len(lengths) + window)
    qs = [torch.randn(c, nq, hd).to(torch.bfloat16) for c in new]
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    batch.seq_lens_host, batch.per_step = list(lengths), {}
    out = torch.full_like(q, float("nan"))
    ops().attention(q, k_pool, v_pool, batch, table, 32, out, nq, nkv, hd, window, hd ** -0.5, workspace=Workspace(DEV))
    assert status.item() == 0
    at = 0
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, hd ** -0.5)
        got = out[at:at + c].double().cpu().reshape(c, nq, hd)
        assert not torch.isnan(got).any(), (s, n, c)
        assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (s, n, c, (got - want).abs().max().item())
        at += c


@pytest.mark.parametrize("page, window, runs", [(8, 0, 1), (8, 600, 3), (16, 1000, 1), (8, 0, 4)])
def test_attention_tcgen05_walks_long_block_tables(page, window, runs):
    """Block tables of some hundred entries (the copying warp keeps a run of them in registers and moves on
    along the table): a long sequence with a short portion, one taken whole, with and without a window (whose
    first key lies far inside the table), in one run of keys and in several."""
    nq, nkv, hd = 8, 2, 128
    lengths, new = [2100, 1300, 70], [140, 1300, 3]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=page + window)
    torch.manual_seed(window + runs)
    qs = [torch.randn(c, nq, hd).to(torch.bfloat16) for c in new]
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full_like(q, float("nan"))
    ops().attention_tcgen05(q, k_pool, v_pool, _Batch(lengths, new, status), table, page, out, nq, nkv, hd, window, hd ** -0.5,
                            n_splits=runs)
    assert status.item() == 0
    at = 0
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, hd ** -0.5)
        got = out[at:at + c].double().cpu().reshape(c, nq, hd)
        assert not torch.isnan(got).any(), (s, n, c)
        assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (s, n, c, (got - want).abs().max().item())
        at += c


def test_attention_tcgen05_finds_a_far_key_and_respects_the_window_edge():
    nq, nkv, hd, page, n = 8, 2, 128, 16, 900
    k_pool, v_pool, table, ks, vs = paged_setup([n], nkv, hd, page, torch.bfloat16, seed=8)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch([n], [40], status)
    for window, target, seen in ((0, 0, True), (0, 63, True), (0, 64, True), (0, 511, True), (0, n - 1, True),
                                 (100, n - 101, False), (100, n - 100, True)):
        q = torch.zeros(40, nq, hd)
        q[:, :, 5] = 24.0
        kp = k_pool.clone()
        kp[table[0, target // page].item(), :, target % page, :] = 0
        kp[table[0, target // page].item(), :, target % page, 5] = 24.0
        out = torch.empty(40, nq * hd, dtype=torch.bfloat16, device=DEV)
        ops().attention_tcgen05(q.reshape(40, -1).to(torch.bfloat16).to(DEV), kp, v_pool, batch, table, page, out, nq, nkv, hd,
                                window, hd ** -0.5)
        want = vs[0][target].float().repeat_interleave(nq // nkv, 0).reshape(-1)
        hit = (out[-1].float().cpu() - want).abs().max().item() < 2e-2     # the last token, at position n - 1
        assert hit == seen, (window, target)
    assert status.item() == 0


@pytest.mark.parametrize("shape", ["rising", "falling", "steps", "wide", "flat"])
@pytest.mark.parametrize("per_block, runs, hd", [(2, 1, 128), (1, 1, 128), (2, 3, 128), (2, 1, 64), (2, 2, 64)])
def test_attention_tcgen05_when_the_reference_has_to_move(shape, per_block, runs, hd):
    """The kernel takes exponentials against a reference that it moves only when a score exceeds it by 2^8: a pair of
    key tiles is tried in one pass and done again where that pass meets a larger score.  Scores that rise with the
    key's position make every pair move the reference (and rescale O); scores that fall never do after the first
    keys; steps move it in the middle of a pair for some rows only; a wide spread mixes all of it; flat scores are
    all equal.  Key j is a multiple of one direction, so the score of (query, key j) is known."""
    nq, nkv, page = 8, 2, 64
    lengths, new = [1500, 333], [330, 333]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=len(shape))
    torch.manual_seed(7)
    direction = torch.nn.functional.normalize(torch.randn(hd), dim=0)
    for s, n in enumerate(lengths):
        j = torch.arange(n, dtype=torch.float32)
        amount = {"rising": j * 0.9, "falling": (n - j) * 0.9, "steps": torch.floor(j / 37.0) * 30.0,
                  "wide": torch.randn(n) * 40.0, "flat": torch.full((n,), 3.0)}[shape]
        keys = (amount[:, None] * direction[None, :] * (hd ** 0.5) / 8.0).to(torch.bfloat16)   # score = amount * |q . direction| / 8
        ks[s] = keys[:, None, :].expand(n, nkv, hd).contiguous()
        for i in range(-(-n // page)):
            rows = keys[i * page:(i + 1) * page].to(DEV)
            k_pool[table[s, i].item(), :, :rows.shape[0]] = rows[None].expand(nkv, rows.shape[0], hd)
    qs = []
    for c in new:
        q = torch.randn(c, nq, hd) * 0.05 + direction * torch.linspace(2.0, 8.0, c)[:, None, None]   # rows of different steepness
        qs.append(q.to(torch.bfloat16))
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full_like(q, float("nan"))
    ops().attention_tcgen05(q, k_pool, v_pool, _Batch(lengths, new, status), table, page, out, nq, nkv, hd, 0, hd ** -0.5,
                            per_block=per_block, n_splits=runs)
    assert status.item() == 0
    at = 0
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), 0, hd ** -0.5)
        got = out[at:at + c].double().cpu().reshape(c, nq, hd)
        assert not torch.isnan(got).any(), (s, n, c)
        assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (shape, s, (got - want).abs().max().item())
        at += c


@pytest.mark.parametrize("nq, nkv, page, norm, write_kv", [(32, 8, 64, True, True), (5, 3, 16, True, True), (4, 4, 8, False, True),
                                                           (6, 2, 32, True, False)])
def test_qk_rope_cache_for_prompt_portions_agrees_with_the_general_kernel(nq, nkv, page, norm, write_kv):
    """Heads of 128 in bfloat16 and a few hundred tokens take a kernel of their own (a warp per token and eight
    heads); the general kernel (a warp per token and head, its own sines) is the reference: a last bit apart."""
    hd, rot = 128, 128
    torch.manual_seed(nq + page)
    lengths, new = [400, 37, 290], [310, 1, 150]
    n_tok = sum(new)
    n_pages = sum(-(-n // page) for n in lengths) + 2
    table = torch.full((3, max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages).tolist()
    for s, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[s, i] = perm.pop()
    pos, sidx = [], []
    for s, (n, c) in enumerate(zip(lengths, new)):
        pos += list(range(n - c, n))
        sidx += [s] * c
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    seq_index = torch.tensor(sidx, dtype=torch.int32, device=DEV)
    qkv = rnd((n_tok, (nq + 2 * nkv) * hd), torch.bfloat16, 1.0, 3)
    qn = (1 + 0.2 * torch.randn(hd)).to(DEV) if norm else None
    kn = (1 + 0.2 * torch.randn(hd)).to(DEV) if norm else None
    inv_freq = (1e6 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV)
    angles = torch.empty(n_tok, rot, device=DEV)
    ops().rope_table(positions, inv_freq, rot, angles)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    results = []
    for table_given in (None, angles):
        k_pool = torch.full((n_pages, nkv, page, hd), 5.0, dtype=torch.bfloat16, device=DEV)
        v_pool = torch.full_like(k_pool, -2.0)
        q_out = torch.full((n_tok, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops().qk_rope_cache(qkv, qn, kn, 1e-6, inv_freq, rot, positions, seq_index, table.to(DEV), page, k_pool, v_pool, q_out,
                            nq, nkv, hd, write_kv, status, cos_sin=table_given)
        results.append((q_out, k_pool, v_pool))
    assert status.item() == 0
    for a, b in zip(*results):
        a, b = a.double(), b.double()
        assert bool(((a - b).abs() <= 2 ** -7 * torch.maximum(a.abs(), b.abs()) + 1e-6).all())
    assert torch.equal(results[0][2], results[1][2])
    assert (results[0][0] == results[1][0]).double().mean().item() > 0.98


@pytest.mark.parametrize("splits", [None, 1, 4, 12])
@pytest.mark.parametrize("nq, nkv, page, norm, write_kv, window", [
    (32, 8, 64, True, True, 0), (16, 1, 16, True, True, 0), (8, 8, 8, False, True, 0), (12, 4, 32, True, False, 0),
    (32, 8, 64, True, True, 100), (8, 2, 16, True, True, 65)])
def test_decoding_attention_that_finishes_the_projection_itself(nq, nkv, page, norm, write_kv, window, splits):
    """One token a sequence, heads of 128: the decoding kernel given the q/k/v rows as the projection leaves them
    (it norms and rotates its token, stores key and value, and puts them into the tile it fetched) against the
    separate kernel followed by the same attention kernel: the same bits in the output and in the pages."""
    from rust_mlx_b200.engine.workspace import Workspace
    hd, rot = 128, 128
    torch.manual_seed(nq * 10 + page)
    lengths = [200, 17, 64, 65, 700, 1, 128]
    new = [1] * len(lengths)
    k0, v0, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=nq + page)
    n = len(lengths)
    positions = torch.tensor([l - 1 for l in lengths], dtype=torch.int32, device=DEV)
    seq_index = torch.arange(n, dtype=torch.int32, device=DEV)
    qkv = rnd((n, (nq + 2 * nkv) * hd), torch.bfloat16, 1.0, 9)
    qn = (1 + 0.2 * torch.randn(hd)).to(DEV) if norm else None
    kn = (1 + 0.2 * torch.randn(hd)).to(DEV) if norm else None
    inv_freq = (1e6 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV)
    angles = torch.empty(n, rot, device=DEV)
    ops().rope_table(positions, inv_freq, rot, angles)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    ws = Workspace(DEV)
    scale = hd ** -0.5
    # separately: the pages get the token's key and value, q its rotated queries; then attention
    k1, v1 = k0.clone(), v0.clone()
    q1 = torch.empty(n, nq * hd, dtype=torch.bfloat16, device=DEV)
    ops().qk_rope_cache(qkv, qn, kn, 1e-6, inv_freq, rot, positions, seq_index, table, page, k1, v1, q1, nq, nkv, hd, write_kv,
                        status, cos_sin=angles)
    out1 = torch.full((n, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops().attention_flash(q1, k1, v1, batch, table, page, out1, nq, nkv, hd, window, scale, ws, n_splits=splits)
    # in one: the token's slot in the pages holds NaN until the kernel stores there
    k2, v2 = k0.clone(), v0.clone()
    if write_kv:
        for s, l in enumerate(lengths):
            k2[table[s, (l - 1) // page], :, (l - 1) % page] = float("nan")
            v2[table[s, (l - 1) // page], :, (l - 1) % page] = float("nan")
    out2 = torch.full_like(out1, float("nan"))
    ops().attention_flash(None, k2, v2, batch, table, page, out2, nq, nkv, hd, window, scale, ws, n_splits=splits,
                          projection=(qkv, qn, kn, 1e-6, angles, write_kv))
    assert status.item() == 0
    assert not torch.isnan(out2.float()).any()
    assert torch.equal(out1, out2)
    # (bit patterns: slots that no request holds are NaN in both)
    assert torch.equal(k1.view(torch.int16), k2.view(torch.int16)) and torch.equal(v1.view(torch.int16), v2.view(torch.int16))


@pytest.mark.parametrize("m, n, k, splits, cluster", [(8, 4096, 4096, 4, True), (8, 1000, 2048, 3, False), (40, 640, 512, 1, True),
                                                      (16, 4096, 12288, 6, True)])
def test_a_wait_that_runs_out_is_reported_and_leaves_the_kernel_usable(m, n, k, splits, cluster):
    """The give-up path of the tcgen05 product: its kernel is launched so that no tile ever arrives and every wait
    on a barrier gives up after 1,000 polls.  It must return (not hang, not trap), report status 3, write nothing,
    free its tensor memory and leave the tiles' split-K counters at zero; the next ordinary product on the same
    stream, with the same scratch, is right."""
    a = rnd((m, k), torch.bfloat16, 1.0, 1)
    w = rnd((n, k), torch.bfloat16, k ** -0.5, 2)
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    counters = ops().gemm_tcgen05_wait_probe(a, w, out, status, splits=splits, cluster=cluster, spin_limit=1000)
    torch.cuda.synchronize()
    assert status.item() == 3
    assert bool((out == 7.0).all())
    if counters is not None:
        assert int(counters.abs().sum().item()) == 0
    status.zero_()
    for _ in range(3):          # tensor memory was given back: blocks of later launches still get theirs
        ops().gemm_tcgen05(a, w, out, status=status, splits=splits, cluster=cluster)
    torch.cuda.synchronize()
    assert status.item() == 0
    want = a.double() @ w.double().t()
    assert (out.double() - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())


def test_the_engine_raises_when_a_kernel_reports_a_wait_that_ran_out(tmp_path):
    """The status word reaches the host: a step after which the word holds 3 raises, commits no lengths, and the
    engine steps on."""
    import tiny
    from rust_mlx_b200.engine import Engine, EngineError
    raw, page = tiny.CONFIGS["D"]
    folder = tiny.make_folder(tmp_path, raw, seed=2)
    eng = Engine(folder, dtype="bfloat16", max_tokens=256, page_size=page, max_requests=2)
    ids = tiny.prompts(raw["vocab_size"], [20], seed=1)[0]
    first = eng.step([("a", ids[:10], [9])]).cpu()
    a = rnd((8, 512), torch.bfloat16, 1.0, 1)
    w = rnd((256, 512), torch.bfloat16, 0.05, 2)
    ops().gemm_tcgen05_wait_probe(a, w, torch.empty(8, 256, dtype=torch.bfloat16, device=DEV), eng._status, splits=2)
    with pytest.raises(EngineError, match="gave up waiting"):
        eng.step([("a", ids[10:], [9])])
    assert eng.length("a") == 10                      # the step was not committed
    again = eng.step([("a", ids[10:], [9])])           # ... and runs when asked again
    eng.release("a")
    whole = eng.step([("b", ids, [9, 19])], ["b"]).cpu()
    assert torch.equal(whole[0], first[0])
    assert (whole[1] - again[0].cpu()).abs().max().item() < 2e-2

"""Seeded random cases: shapes, lengths, page sizes, windows and ways of cutting that nobody picked by hand.

Each test draws its cases from a fixed seed, so a failure names a case that can be run again.  The
bounds are those of the hand-picked tests of the same kernels and paths.
"""
import random

import pytest
import torch

import plain_qwen3 as plain
import replay
import tiny
from test_kernels_gpu import DEV, _Batch, ops, paged_setup, plain_attention

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_attention_of_random_steps(seed):
    """``ops.attention`` (which picks the kernels and divides mixed steps) over random head sizes, groups, page
    sizes, windows and mixes of decoded tokens, short and long portions, in bfloat16."""
    from rust_mlx_b200.engine.workspace import Workspace
    rng = random.Random(seed)
    ws = Workspace(DEV)
    done = 0
    while done < 60:
        hd = rng.choice([16, 32, 64, 96, 128, 128, 128])
        nkv, group = rng.choice([1, 2, 3, 8]), rng.choice([1, 2, 3, 4, 8])
        nq = nkv * group
        page, window = rng.choice([8, 16, 32, 64, 128]), rng.choice([0, 0, 17, 100, 700])
        lengths, new = [], []
        for _ in range(rng.randint(1, 6)):
            n = rng.choice([1, 2, 17, 63, 64, 65, 129, 300, 700, 1500])
            lengths.append(n)
            new.append(min(n, rng.choice([1, 1, 1, 2, 5, 16, 33, 64, 130, 400, n])))
        if not ops().flash_supported(hd, group):
            continue
        done += 1
        k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.bfloat16, seed=done)
        torch.manual_seed(done)
        qs = [torch.randn(c, nq, hd).to(torch.bfloat16) for c in new]
        q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        batch = _Batch(lengths, new, status)
        batch.seq_lens_host, batch.per_step = list(lengths), {}
        out = torch.full_like(q, float("nan"))
        ops().attention(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, window, hd ** -0.5, workspace=ws)
        case = (seed, done, hd, nq, nkv, page, window, lengths, new)
        assert status.item() == 0, case
        at = 0
        for s, (n, c) in enumerate(zip(lengths, new)):
            want = plain_attention(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, hd ** -0.5)
            got = out[at:at + c].double().cpu().reshape(c, nq, hd)
            assert not torch.isnan(got).any(), (case, s)
            assert ((got - want).abs() <= 1e-2 * (1 + want.abs())).all(), (case, s, (got - want).abs().max().item())
            at += c


@pytest.mark.parametrize("seed", [1, 2])
def test_tcgen05_products_of_random_shapes(seed):
    """The tcgen05 product over random row counts, widths that are no multiple of a tile, reductions that are no
    multiple of a k block, numbers of K slices, float and bfloat16 results, with and without the SwiGLU epilogue."""
    rng = random.Random(seed)
    done = 0
    while done < 80:
        m = rng.choice([1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 48, 63, 64])
        n = rng.choice([8, 64, 128, 136, 200, 509, 1000, 1024, 4096, 6144, 333, 2056])
        k = rng.choice([8, 64, 72, 128, 136, 256, 520, 1024, 4096, 2056])
        swiglu = rng.random() < 0.3 and n % 128 == 0
        splits = rng.choice([None, 1, 2, 3, 4, 5, 8])
        if splits is not None and splits > max(1, -(-k // 64)):
            continue
        done += 1
        torch.manual_seed(done)
        a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
        w = (torch.randn(n, k, device=DEV) * 0.05).to(torch.bfloat16)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ref = a.double() @ w.double().t()
        if swiglu:
            out = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops().gemm_tcgen05(a, w, out, status=status, swiglu=True)
            r = ref.view(m, n // 128, 2, 64)
            want, tol = (r[:, :, 0] / (1 + torch.exp(-r[:, :, 0])) * r[:, :, 1]).reshape(m, n // 2), 2e-2
        else:
            odt = rng.choice([torch.float32, torch.bfloat16])
            out = torch.full((m, n), float("nan"), dtype=odt, device=DEV)
            ops().gemm_tcgen05(a, w, out, status=status, splits=splits)
            want, tol = ref, (2e-2 if odt == torch.bfloat16 else 2e-3)
        err = ((out.double() - want).abs() / (1 + want.abs())).max().item()
        assert status.item() == 0 and err < tol, (seed, done, m, n, k, splits, swiglu, err)


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    return tmp_path_factory.mktemp("fuzz")


@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106, 107, 108])
def test_replay_of_random_requests_cut_at_random(workdir, seed):
    """A random configuration of the five, random request lengths up to 1,500 tokens, random cuts with up to four
    requests in a step, in a cache that holds what the trace needs and no more.  float32: within 1e-4 of the plain
    implementation and the very bits each request gives alone and whole.  bfloat16: as close to the plain
    implementation restated with bfloat16 roundings as that restatement is to the exact logits (at least 2e-2)."""
    from rust_mlx_b200.engine import Engine
    rng = random.Random(seed)
    name = rng.choice(["A", "B", "Bw", "C", "D", "E"])
    raw, page = tiny.CONFIGS[name]
    sub = workdir / str(seed)
    sub.mkdir()
    folder = tiny.sharpen(tiny.make_folder(sub, raw, seed=seed, store="float32"))
    lens = [rng.choice([1, 2, 5, 31, 64, 65, 128, 200, 333, 500, 777, 1500]) for _ in range(rng.randint(2, 6))]
    reqs = {f"q{i}": p for i, p in enumerate(tiny.prompts(raw["vocab_size"], lens, seed=seed))}
    steps = replay.random_cuts(reqs, seed, live=rng.randint(1, 4), largest=rng.choice([40, 300, 700]))
    exact = plain.PlainModel(folder)
    for dtype in ("float32", "bfloat16"):
        pm = exact if dtype == "float32" else plain.PlainModel(folder, rounding="bfloat16")
        eng = Engine(folder, dtype=dtype, max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        assert eng.pools.table.live() == 0
        for rid, toks in reqs.items():
            want = pm.logits(toks).float()
            bound = 1e-4 if dtype == "float32" else max(2e-2, tiny.max_abs(want, exact.logits(toks).float()))
            assert tiny.max_abs(got[rid], want) < bound, (seed, name, dtype, rid, len(toks), bound)
        if dtype == "float32":
            alone = replay.run_engine(Engine(folder, dtype=dtype, max_tokens=max(-(-n // page) * page for n in lens),
                                             page_size=page, max_requests=4), replay.whole(reqs))
            for rid in reqs:
                assert torch.equal(got[rid], alone[rid]), (seed, name, rid)

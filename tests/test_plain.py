"""The plain implementation's parts, checked against properties that do not depend on it (no GPU)."""
import math

import torch

import plain_qwen3 as plain
import tiny

F = torch.float64


def test_rms_norm_by_hand():
    v = torch.tensor([[3.0, 4.0]], dtype=F)
    w = torch.tensor([2.0, 0.5], dtype=F)
    out = plain.rms_norm(v, w, 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]], dtype=F))


def test_rope_is_a_rotation_of_half_split_pairs():
    torch.manual_seed(0)
    x = torch.randn(5, 3, 8, dtype=F)
    pos = torch.tensor([0, 1, 2, 10, 100])
    y = plain.rope(x, pos, 10000.0, 8)
    assert torch.equal(y[0], x[0])                                  # position 0: nothing moves
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))           # lengths are kept
    # pair (j, j + half) turns by pos * theta^(-2j/dim)
    j, t = 1, 3
    ang = float(torch.tensor(10.0) * torch.tensor(10000.0 ** (-2 * j / 8), dtype=torch.float32))
    a, b = x[t, 0, j], x[t, 0, j + 4]
    assert torch.allclose(y[t, 0, j], a * math.cos(ang) - b * math.sin(ang))
    assert torch.allclose(y[t, 0, j + 4], b * math.cos(ang) + a * math.sin(ang))
    # scores depend on the distance of positions only
    q, k = torch.randn(1, 1, 8, dtype=F), torch.randn(1, 1, 8, dtype=F)
    s1 = (plain.rope(q, torch.tensor([7]), 1e4, 8) * plain.rope(k, torch.tensor([3]), 1e4, 8)).sum()
    s2 = (plain.rope(q, torch.tensor([104]), 1e4, 8) * plain.rope(k, torch.tensor([100]), 1e4, 8)).sum()
    assert torch.allclose(s1, s2, atol=1e-4)   # angles are float32 products
    # partial rotation leaves the rest alone
    z = plain.rope(x, pos, 1e4, 4)
    assert torch.equal(z[..., 4:], x[..., 4:])


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(1)
    T, nq, nkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=F) for n in (nq, nkv, nkv))
    pos = torch.arange(T)
    out = plain.attention_scores(q, k, v, pos, 0)
    # the first token sees itself only
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])
    # later keys do not matter
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0, 0
    assert torch.allclose(plain.attention_scores(q, k2, v2, pos, 0)[:5], out[:5])
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v3 = v.clone()
    v3[:, 1] += 1.0
    out3 = plain.attention_scores(q, k, v3, pos, 0)
    assert torch.allclose(out3[:, :2], out[:, :2]) and torch.allclose(out3[:, 2:], out[:, 2:] + 1.0)
    # a window of 3: token 8 sees keys 6, 7, 8
    w = plain.attention_scores(q, k, v, pos, 3)
    s = (q[8, 0] @ k[6:9, 0].t()) * hd ** -0.5
    assert torch.allclose(w[8, 0], torch.softmax(s, -1) @ v[6:9, 0])
    assert torch.allclose(w[:3], out[:3])


def test_swiglu_by_hand():
    w = {"m.gate_proj.weight": torch.tensor([[1.0, 0.0]], dtype=F), "m.up_proj.weight": torch.tensor([[0.0, 2.0]], dtype=F),
         "m.down_proj.weight": torch.tensor([[1.0], [-1.0]], dtype=F)}
    x = torch.tensor([[0.5, 3.0]], dtype=F)
    g = 0.5
    act = g / (1 + math.exp(-g)) * 6.0
    out = plain.swiglu_mlp(x, w, "m", lambda t: t)
    assert torch.allclose(out, torch.tensor([[act, -act]], dtype=F))


def test_whole_model_is_causal_and_tied_head_reads_the_embedding(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_A, seed=2)
    m = plain.PlainModel(folder)
    ids = tiny.prompts(256, [12])[0]
    full = m.logits(ids)
    assert full.shape == (12, 256)
    assert torch.allclose(m.logits(ids[:7]), full[:7], atol=1e-12)
    assert "lm_head.weight" not in m.w


def test_window_changes_only_late_positions(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_BW, seed=2)
    m = plain.PlainModel(folder)
    ids = tiny.prompts(509, [30])[0]
    with_window = m.logits(ids)
    m.config["use_sliding_window"] = False
    without = m.logits(ids)
    assert torch.allclose(with_window[:20], without[:20], atol=1e-12)     # window 20 not yet felt
    assert (with_window[25:] - without[25:]).abs().max() > 1e-6


def test_bfloat16_restatement_is_close_but_not_equal(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_A, seed=2)
    ids = tiny.prompts(256, [10])[0]
    a = plain.PlainModel(folder).logits(ids)
    b = plain.PlainModel(folder, rounding="bfloat16").logits(ids)
    d = (a - b).abs().max().item()
    assert 1e-5 < d < 5e-2

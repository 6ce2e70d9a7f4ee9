"""Writes tests/golden/dense_fixture_plain.json: what tests/plain_qwen3.py gives for the
reference's fixture (tests/fixtures/dense of d9beuD/rust-mlx), beside the oracle's own
numbers.  The reference's model code cannot run here (no Rust, no MLX); its shipped
oracle.json is the comparison.  Run from the repository root:
    python tests/golden/make_dense_fixture_plain.py /path/to/reference/tests/fixtures/dense
"""
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
import plain_qwen3 as plain  # noqa: E402

fixture = sys.argv[1]
oracle = json.load(open(os.path.join(fixture, "oracle.json")))
m = plain.PlainModel(fixture)
logits = m.logits(oracle["prompt"])[-1]
tokens = m.greedy(oracle["prompt"], len(oracle["tokens"]))
err = max(abs(a - b) for a, b in zip(logits.tolist(), oracle["prefill_logits"]))
out = {"prompt": oracle["prompt"], "tokens": tokens, "last_logits": logits.tolist(),
       "oracle_tokens_equal": tokens == oracle["tokens"], "max_abs_vs_oracle": err}
json.dump(out, open(os.path.join(os.path.dirname(__file__), "dense_fixture_plain.json"), "w"))
print("tokens equal:", out["oracle_tokens_equal"], "max abs vs oracle:", err)

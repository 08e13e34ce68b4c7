"""Writes tests/golden/kcheck_vectors.json: the power-law exponent that the reference's Python
prototype of the k-check fits to a best-first list of attention weights
(`fit_powerlaw_alpha_from_head`, tools/analyze_attn_samples.ipynb, code cell 5 — the function the
Rust `fit_alpha_from_logits`, diffcache_cpu/src/nsw.rs:198-240, re-implements: least-squares slope of
log-weight against log-rank from rank 5 on).

Only that function definition is taken out of the notebook (by `ast`, unmodified) and executed; the
rest of the cell reads a sample file that is not part of the checkout.  The inputs are seeded lists
of ranking keys `bits(65536 - dot)` as the engine produces them; the prototype receives
exp(dot / sqrt(D)), the weights it is written for (sorted descending).

Run from the repository root:
    python tests/golden/make_kcheck_vectors.py /path/to/DiffCache
"""
import ast
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.util import KCHECK_CASES, kcheck_case_bits  # noqa: E402


def load_prototype(ref):
    path = os.path.join(ref, "tools", "analyze_attn_samples.ipynb")
    if not os.path.isfile(path):
        raise SystemExit("usage: make_kcheck_vectors.py <DiffCache checkout>")
    with open(path) as f:
        cell = "".join(json.load(f)["cells"][5]["source"])
    tree = ast.parse(cell)
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "fit_powerlaw_alpha_from_head"]
    assert len(fn) == 1
    ns = {"np": np, "torch": torch}
    exec(compile(ast.Module(body=fn, type_ignores=[]), path, "exec"), ns)
    return ns["fit_powerlaw_alpha_from_head"]


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DIFFCACHE_REFERENCE", "")
    fit = load_prototype(ref)
    out = {}
    for name, case in KCHECK_CASES.items():
        bits = kcheck_case_bits(case)
        dist = bits.view(np.float32).astype(np.float64)
        logits = (65536.0 - dist) / np.sqrt(float(case["head_dim"]))      # nsw.rs:287-290
        weights = torch.from_numpy(np.exp(logits - logits.max()))         # a common factor does not move the slope
        alpha = fit(weights, i_min=5)
        out[name] = {"alpha": alpha, "n": int(bits.shape[0])}
        print(name, out[name])
    with open(os.path.join(HERE, "kcheck_vectors.json"), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()

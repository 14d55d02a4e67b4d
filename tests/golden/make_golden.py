"""Regenerates tests/golden/golden.npz from the COMPILED REFERENCE (oracle/_ref, i.e. the
reference's own kernels/compact_counter.cl built by oracle/Makefile).

Run from the repository root where the reference tree is mounted:
    python tests/golden/make_golden.py
For every case of cases.py it stores the reference outputs of: decode_weight, the dense
update (fed the r-ascending fp32 dY^T X), the memory-native fused update and
backward_input (dense float outputs only for the small cases).  A SHA-256 of each case's inputs is stored too, so the tests notice if the
input generators drift.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import oracle  # noqa: E402
from cases import all_cases  # noqa: E402


def digest(case) -> str:
    h = hashlib.sha256()
    for k in ("state", "scale", "v", "x", "dy"):
        h.update(np.ascontiguousarray(case[k]).tobytes())
    return h.hexdigest()


def main():
    oracle.build()
    import importlib
    importlib.reload(oracle)
    ref = oracle.ref
    assert ref is not None, "compiled reference not available"
    out = {}
    for c in all_cases():
        n, I, O, C = c["name"], c["I"], c["O"], c["C"]
        hy = (c["lr"], c["lr_scale"], c["beta"], c["eps"], c["seed"])
        out[f"{n}/digest"] = np.frombuffer(bytes.fromhex(digest(c)), np.uint8)
        small = O * I < 10000     # dense float outputs are kept for the small cases only
        if small:
            out[f"{n}/weight"] = ref.decode_weight(c["state"], c["scale"], C, I, O)
        gw = oracle.port.grad_w(c["dy"], c["x"])   # r-ascending fp32 dY^T X (validated below)
        st, sc, v = ref.update_dense(c["state"], c["scale"], c["v"], gw, C, I, O, *hy)
        out[f"{n}/dense_state"], out[f"{n}/dense_scale"], out[f"{n}/dense_v"] = st, sc, v
        st2, sc2, v2 = ref.update_fused(c["state"], c["scale"], c["v"], c["dy"], c["x"], C, *hy)
        # the fused kernels recompute exactly that gradient, so both reference paths agree
        assert (st == st2).all() and (sc == sc2).all() and (v == v2).all(), n
        if small:
            out[f"{n}/grad_x"] = ref.backward_input(c["dy"], c["state"], c["scale"], C, I)
        print(n, "state bytes changed:", float((st != c["state"]).mean()))
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz"), **out)


if __name__ == "__main__":
    main()

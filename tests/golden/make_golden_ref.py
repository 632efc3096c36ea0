"""Record golden vectors from the reference's own kernels.  Run on a machine with a B200 and the
prebuilt oracle/_ref/cdssm_ref_C.so (python oracle/build_ref.py builds it where the reference
sources are mounted):

    python tests/golden/make_golden_ref.py [outdir]

Writes ref_<case>.npz files and bwd_ref.npz (the reference's backward kernels on one small case) (default: ./golden_out/); copy them into tests/golden/.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))


def main():
    import oracle
    from oracle.build_ref import load_ref
    from golden.golden_cases import CASES, run_reference, run_reference_backward
    ref = load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/cdssm_ref_C.so not built")
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "golden_out")
    os.makedirs(out, exist_ok=True)
    for name, case in CASES.items():
        res = run_reference(ref, case, oracle)
        path = os.path.join(out, f"ref_{name}.npz")
        np.savez_compressed(path, **res)
        print(name, {k: v.shape for k, v in res.items() if hasattr(v, "shape") and v.ndim > 1},
              os.path.getsize(path), "bytes")
    path = os.path.join(out, "bwd_ref.npz")
    np.savez_compressed(path, **run_reference_backward(ref, oracle))
    print("backward", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

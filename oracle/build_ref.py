"""Compile the reference's own CUDA extension (unmodified sources, read where they lie)
into oracle/_ref/ so that GPU tests can pin the oracle against the real kernels.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file or its output.

The reference ships only `-gencode arch=compute_90,code=sm_90` (setup.py:41-47), which
cannot load on a B200, so the same sources are compiled here for sm_100 with the
reference's other flags (`-O3 --use_fast_math`).  The result is a torch extension
module `cdssm_ref_C` exposing the twelve `*_cuda` functions of cdssm/csrc/binding.cpp:130-202.

Usage:  python oracle/build_ref.py [reference_root]   (default: $CDSSM_REFERENCE_ROOT, else a checkout named
`reference` beside this repository)
The sources are never copied into this repository; only the built `.so` lands in
oracle/_ref/ (git-ignored).
"""
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
KERNELS = ["conv1d_silu.cu", "dynamics_fused.cu", "intra_chunk_scan.cu",
           "inter_chunk_scan.cu", "exact_correction.cu", "normalize_kq.cu"]


def ref_so_path():
    return os.path.join(OUT, "cdssm_ref_C.so")


def default_reference_root():
    """$CDSSM_REFERENCE_ROOT, else a checkout named ``reference`` beside this repository, else None."""
    env = os.environ.get("CDSSM_REFERENCE_ROOT")
    if env:
        return env
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return beside if os.path.isdir(beside) else None


def build(reference_root=None, verbose=False):
    reference_root = reference_root or default_reference_root()
    if not reference_root:
        raise FileNotFoundError("no reference checkout: set CDSSM_REFERENCE_ROOT")
    csrc = os.path.join(reference_root, "cdssm", "csrc")
    if not os.path.isdir(csrc):
        raise FileNotFoundError(f"reference sources not found under {reference_root}")
    if os.path.exists(ref_so_path()):
        return ref_so_path()
    from torch.utils.cpp_extension import load
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    srcs = [os.path.join(csrc, "binding.cpp")] + [os.path.join(csrc, "kernels", k) for k in KERNELS]
    t0 = time.time()
    load(name="cdssm_ref_C", sources=srcs,
         extra_include_paths=[os.path.join(csrc, "include")],
         extra_cflags=["-O3"],
         extra_cuda_cflags=["-O3", "--use_fast_math", "-gencode", "arch=compute_100,code=sm_100",
                            "--threads", "4"],
         build_directory=OUT, verbose=verbose, is_python_module=False)
    print(f"built {ref_so_path()} in {time.time() - t0:.0f}s")
    return ref_so_path()


def load_ref():
    """Import the prebuilt module (no sources needed).  Returns None if it was never built."""
    p = ref_so_path()
    if not os.path.exists(p):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch symbols must be loaded first)
    spec = importlib.util.spec_from_file_location("cdssm_ref_C", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    build(*(sys.argv[1:2]), verbose=True)

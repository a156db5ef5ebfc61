"""Build the reference's own CUDA kernels for the hot path into oracle/_ref/ (git-ignored).

Test infrastructure only.  The reference (microsoft/Swin3D) ships its all-in-one attention
kernels in Swin3D/src/attn/self_attn_aio_{fwd,bwd}.cu and its KNN in
Swin3D/src/knn/knn_cuda_kernel.cu.  They do not compile against torch >= 2.x as they are,
because seven AT_DISPATCH_FLOATING_TYPES_AND_HALF call sites pass `tensor.type()` where a
ScalarType is required.  This recipe copies those few files to a scratch directory outside
the repository, rewrites `.type()` to `.scalar_type()` at exactly those call sites, and
compiles them (nvcc, no GPU needed) together with oracle/ref_binding/ref_aio_api.cpp into
oracle/_ref/ref_swin3d_cuda.so.  No reference source is written into this repository.

Usage:  python oracle/build_ref.py [--reference /path/to/Swin3D-checkout]   (default: $SWIN3D_REFERENCE,
        else a directory `reference` beside this repository)
The product never loads the result; only tests/ and bench.py's reference-kernel timing do.

Safe-use note for callers: the reference forward kernel keeps a `__shared__ scalar_t[32]`
staging array indexed by (threadIdx.x / (head_dim / pack)) with 512 threads
(self_attn_aio_fwd.cu:166-176).  That index stays below 32 only when head_dim/pack >= 16,
i.e. fp32/fp64 with head_dim >= 16 and fp16 with head_dim == 32.  The tests therefore call the
reference forward only with those shapes; other shapes would index past the array.
"""
import argparse
import os
import re
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "ref_swin3d_cuda"

ATTN_FILES = ["self_attn_aio_fwd.cu", "self_attn_aio_fwd.h", "self_attn_aio_bwd.cu",
              "self_attn_aio_bwd.h", "attn_utils.cuh", "torch_utils.h"]
KNN_FILES = ["knn_cuda_kernel.cu", "knn_cuda_kernel.h", "cuda_utils.cuh", "torch_utils.h"]


def default_reference_root() -> str:
    """$SWIN3D_REFERENCE, else a directory `reference` beside this repository."""
    env = os.environ.get("SWIN3D_REFERENCE")
    return env if env else os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def stage_sources(ref_root: str, scratch: str):
    pat = re.compile(r"(AT_DISPATCH_FLOATING_TYPES_AND_HALF\(\s*\w+)\.type\(\)")
    for sub, files in (("attn", ATTN_FILES), ("knn", KNN_FILES)):
        os.makedirs(os.path.join(scratch, sub), exist_ok=True)
        for f in files:
            src = os.path.join(ref_root, "Swin3D", "src", sub, f)
            with open(src, "r") as fh:
                text = fh.read()
            text = pat.sub(r"\1.scalar_type()", text)
            with open(os.path.join(scratch, sub, f), "w") as fh:
                fh.write(text)


def build(ref_root: str, verbose: bool = True) -> str:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load
    os.makedirs(OUT, exist_ok=True)
    scratch = tempfile.mkdtemp(prefix="swin3d_ref_src_")
    try:
        stage_sources(ref_root, scratch)
        binding = os.path.join(scratch, "ref_aio_api.cpp")
        shutil.copy(os.path.join(HERE, "ref_binding", "ref_aio_api.cpp"), binding)
        load(name=NAME,
             sources=[binding,
                      os.path.join(scratch, "attn", "self_attn_aio_fwd.cu"),
                      os.path.join(scratch, "attn", "self_attn_aio_bwd.cu"),
                      os.path.join(scratch, "knn", "knn_cuda_kernel.cu")],
             extra_include_paths=[scratch],
             extra_cflags=["-O2"],
             extra_cuda_cflags=["-O2"],
             build_directory=OUT, verbose=verbose, is_python_module=False)
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return os.path.join(OUT, NAME + ".so")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference_root(),
                    help="checkout of microsoft/Swin3D (default: $SWIN3D_REFERENCE, else ../reference beside this repository)")
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(a.reference, "Swin3D", "src", "attn")):
        print("reference checkout not found at", a.reference, "- nothing built")
        sys.exit(0)
    print(build(a.reference))

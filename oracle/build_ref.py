"""Builds the reference's own page-copy kernel into oracle/_ref/.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [path-to-Bi-KV-checkout]

Compiles ``SharedMemory/CUDA_Shared/copy_kernel.cu`` from the checkout, unmodified and in
place, together with ``oracle/ref_harness.cpp`` for sm_100a (torch's extension builder;
no GPU needed).  The result, ``oracle/_ref/bikv_ref_kernel.so``, is git-ignored and is
used by the GPU tests as a second, independent checker and by nothing else.  Without a
checkout this script does nothing and exits 0.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "bikv_ref_kernel"


def main() -> int:
    # The reference checkout: first argument, else $BIKV_REFERENCE_ROOT, else a directory named
    # "reference" beside this repository.
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BIKV_REFERENCE_ROOT") or \
        os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    src_dir = os.path.join(root, "Bi-KV", "SharedMemory", "CUDA_Shared")
    kernel = os.path.join(src_dir, "copy_kernel.cu")
    if not os.path.exists(kernel):
        print(f"no reference checkout at {root}: nothing built")
        return 0
    target = os.path.join(OUT, NAME + ".so")
    harness = os.path.join(HERE, "ref_harness.cpp")
    if os.path.exists(target) and os.path.getmtime(target) > max(os.path.getmtime(kernel), os.path.getmtime(harness)):
        print(f"{target} is up to date")
        return 0
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load

    load(name=NAME, sources=[harness, kernel], extra_include_paths=[src_dir], build_directory=OUT,
         extra_cflags=["-O2"], extra_cuda_cflags=["-O3", "-lineinfo"], extra_ldflags=["-lrt", "-lpthread"],
         with_cuda=True, is_python_module=False, verbose=False)
    print(f"built {target}")
    return 0


if __name__ == "__main__":
    sys.exit(main())

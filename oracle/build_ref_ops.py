"""Oracle build of the reference's own CUDA MoE ops.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref_ops.py /path/to/electrock-infer
    ELECTROCK_REFERENCE=/path/to/electrock-infer python oracle/build_ref_ops.py

Compiles, from where they lie in the reference source tree and without modifying or copying them,
src/{topk_softmax_kernels,moe_align_block_size,activation_kernels,moe_sum,moe_sum_efficient}.cu
with nvcc for sm_100a, together with the small binding ``ref_ops_binding.cpp`` kept beside this
script, into ``oracle/_ref/ref_ops*.so`` (git-ignored).  ``ref_shim/cuda_utils.cuh`` stands in for
the reference header of the same name, which targets another vendor's runtime; it defines
``WARP_SIZE 32``.  GPU tests import the result when it exists and compare the reference kernels
with libb200moe bit for bit; nothing in the product package knows about it.

Known limits of the reference kernels that the tests respect: ``topk_softmax`` reads past the end
of its input unless the token count is a multiple of 4 (src/topk_softmax_kernels.cu:18), and
``moe_sum_efficient`` has no bf16 instantiation.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
SOURCES = ["topk_softmax_kernels.cu", "moe_align_block_size.cu", "activation_kernels.cu",
           "moe_sum.cu", "moe_sum_efficient.cu"]


def main() -> int:
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ELECTROCK_REFERENCE")
    if not where:
        print("give the path of the electrock-infer source tree as the first argument or in "
              "ELECTROCK_REFERENCE; nothing built")
        return 2
    ref_root = Path(where)
    src_dir = ref_root / "src"
    if not all((src_dir / s).exists() for s in SOURCES):
        print(f"reference sources not found under {src_dir}; nothing built")
        return 0
    import pybind11
    import torch
    from torch.utils import cpp_extension

    OUT_DIR.mkdir(exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = OUT_DIR / f"ref_ops{ext}"
    inputs = [src_dir / s for s in SOURCES] + [HERE / "ref_ops_binding.cpp",
                                                HERE / "ref_shim" / "cuda_utils.cuh"]
    if target.exists() and all(target.stat().st_mtime > p.stat().st_mtime for p in inputs):
        print(f"up to date: {target}")
        return 0
    includes = [str(HERE / "ref_shim"), str(src_dir / "include"), pybind11.get_include(),
                sysconfig.get_paths()["include"], *cpp_extension.include_paths("cuda")]
    torch_lib = Path(torch.__file__).parent / "lib"
    objs = []
    common = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-DTORCH_EXTENSION_NAME=ref_ops",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
              *[f"-I{i}" for i in includes]]
    procs = []
    for p in inputs[:-1]:
        obj = OUT_DIR / (p.stem + ".o")
        objs.append(obj)
        extra = ["-x", "cu"] if p.suffix == ".cpp" else []
        procs.append((p, subprocess.Popen([*common, *extra, "-c", str(p), "-o", str(obj)],
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                          text=True)))
    for p, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            print(out[-4000:])
            print(f"failed to compile {p}")
            return 1
    link = ["nvcc", "-shared", "-o", str(target), *map(str, objs), f"-L{torch_lib}",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            f"-Xlinker=-rpath={torch_lib}"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        print(proc.stdout[-2000:], proc.stderr[-2000:])
        return 1
    for o in objs:
        o.unlink()
    print(f"built {target}")
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Build libmx8.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python gpu-experiments_b200/build.py [--force] [-v]

Objects go to gpu-experiments_b200/build/, the library to gpu-experiments_b200/mx8/libmx8.so.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "mx8")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(OUT_DIR, "libmx8.so")
SOURCES = ["mx8_host.cu", "quantize.cu", "gemm.cu", "moe_schedule.cu", "moe_combine.cu", "moe_layer.cu", "host_pipeline.cu", "shared_expert.cu", "peak_probe.cu"]
HEADERS = ["mx8_host.cuh", "mx8_ptx.cuh", "mx8_qmath.cuh", os.path.join("..", "..", "include", "mx8.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd))
            subprocess.check_call(cmd)
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "--cudart", "shared", "-Xlinker", "-rpath,/usr/local/cuda/lib64", "-o", LIB] + objs
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return LIB


def torch_binding_path():
    import sysconfig
    return os.path.join(OUT_DIR, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_torch_binding(force=False, verbose=False):
    """Compile csrc/torch_binding.cpp into the pybind11/torch module mx8/_C (links libmx8.so)."""
    import sysconfig

    from torch.utils import cpp_extension as ce
    build(force=False, verbose=verbose)
    src = os.path.join(CSRC, "torch_binding.cpp")
    out = torch_binding_path()
    if not (force or _stale(out, [src, os.path.join(HERE, "..", "include", "mx8.h"), LIB])):
        return out
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    libdirs = ce.library_paths()
    cmd = (["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
            src, "-o", out] + ["-I" + i for i in inc] + ["-L" + d for d in libdirs]
           + ["-L" + OUT_DIR, "-lmx8", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-Wl,-rpath,$ORIGIN"]
           + ["-Wl,-rpath," + d for d in libdirs])
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch_binding(force="--force" in sys.argv, verbose="-v" in sys.argv))

"""Builds csrc/*.cu into libq35b200.so (in-tree, sm_100a only) with nvcc, and the native by-name runner
runner/q35run.cc (plain C++ against the library's C ABI and the CUDA runtime) into ./q35run.

    python -m ax_dsl_kernels_b200.build [--force]
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libq35b200.so")
RUNNER = os.path.join(HERE, "q35run")
RUNNER_SRC = os.path.join(HERE, "runner", "q35run.cc")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-I", os.path.join(os.path.dirname(HERE), "include")]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    cmd = [NVCC, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "q35b200.h"))
    todo = [s for s in sources()
            if force or _stale(os.path.join(OBJ, s[:-3] + ".o"), [os.path.join(CSRC, s), *headers])]
    if verbose and todo:
        print("nvcc:", " ".join(todo), flush=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as ex:
        list(ex.map(_compile, todo))
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources()]
    if todo or _stale(LIB, objs):
        r = subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if force or _stale(RUNNER, [RUNNER_SRC, LIB, headers[-1]]):
        r = subprocess.run([NVCC, "-O2", "-std=c++17", "-I", os.path.join(os.path.dirname(HERE), "include"), RUNNER_SRC,
                            "-o", RUNNER, "-L", HERE, "-lq35b200", "-lcudart", "-lpthread", "-Xlinker", "-rpath", "-Xlinker",
                            "$ORIGIN"], capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"runner build failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))

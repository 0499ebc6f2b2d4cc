"""In-tree build of the CUDA library (sm_100a only) and, where a checkout of the
reference is present, of the reference's own unmodified test / benchmark drivers
linked against this library instead of the reference's kernels.

    python llm-sys-project_b200/build.py            # library (+ drivers when possible)

Outputs: ``llm-sys-project_b200/lib/libb200moedsa.so`` and ``oracle/_ref/drivers/*``
(both git-ignored; they travel with the working tree).
"""
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(LIBDIR, "libb200moedsa.so")

SOURCES = ["runtime.cu", "moe_route.cu", "moe_route_tc.cu", "moe_f32.cu", "moe_fp8.cu", "moe_ep.cu", "dsa_f32.cu", "dsa_bf16.cu", "dsa_bf16_pair.cu",
           "umma_selftest.cu", "wait_selftest.cu", "mx_selftest.cu", "ref_shims.cu"]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
          "--expt-relaxed-constexpr"]


def _host_cxx():
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "b200_moe_dsa.h"))
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJDIR, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + headers):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [NVCC, "-ccbin", _host_cxx()] + ARCH + CFLAGS + ["-c", s, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return s, r

    logs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for s, r in ex.map(compile_one, jobs):
            logs.append((s, r.stderr))
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError(f"nvcc failed on {s}")
            if verbose:
                sys.stderr.write(r.stderr)
    with open(os.path.join(OBJDIR, "ptxas.log"), "a" if not force else "w") as f:
        for s, log in logs:
            f.write(f"==== {os.path.basename(s)}\n{log}\n")
    if jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-ccbin", _host_cxx()] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


def find_reference():
    for p in (os.environ.get("B200_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference"),
              os.path.join(ROOT, "baseline", "_ref")):
        if p and os.path.exists(os.path.join(p, "tests", "test_moe.cu")):
            return p
    return None


def build_reference_drivers(force=False):
    """Compile the reference's tests/ and benchmarks/ drivers, unmodified and from where
    they lie, against this library (its C++ shims carry the reference's symbol names)."""
    ref = find_reference()
    outdir = os.path.join(ROOT, "oracle", "_ref", "drivers")
    if ref is None:
        return None
    os.makedirs(outdir, exist_ok=True)
    built = []
    for rel in ("tests/test_moe.cu", "tests/test_dsa.cu", "benchmarks/bench_moe.cu", "benchmarks/bench_dsa.cu"):
        src = os.path.join(ref, rel)
        exe = os.path.join(outdir, os.path.basename(rel)[:-3])
        if force or _newer(exe, [src, LIB]):
            cmd = [NVCC, "-ccbin", _host_cxx(), "-std=c++17", "-O2"] + ARCH + ["-o", exe, src, "-L" + LIBDIR,
                   "-lb200moedsa", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../llm-sys-project_b200/lib"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError(f"building reference driver {rel} failed")
        built.append(exe)
    return built


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_reference_drivers(force="--force" in sys.argv))

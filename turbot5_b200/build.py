"""Compile the CUDA sources in `csrc/` into `libturbot5_b200.so` next to this file.

    python -m turbot5_b200.build [--force]

The library is built for sm_100a only, in-tree, with nvcc (no JIT cache, no
torch extension machinery: the ABI is plain C, see include/turbot5_b200.h).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libturbot5_b200.so")
SOURCES = ["api.cu", "bucket.cu", "attn_fwd_sm100.cu", "attn_fwd2_sm100.cu", "attn_bwd_sm100.cu", "attn_fwd_simt.cu", "attn_bwd_simt.cu", "decode.cu",
           "rmsnorm.cu", "padding.cu", "fused_ops.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "turbot5_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Build the shared library if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [_nvcc(), "-Xptxas=-v", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose and out:
            sys.stderr.write(out.decode())
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out.decode()}")
        with open(_ptxas_log(src), "w") as f:      # registers and spills per kernel, see resource_report()
            f.write(out.decode())
    tmp = LIB + ".tmp"
    link = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp, *objs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout.decode())
    os.replace(tmp, LIB)
    return LIB


def _ptxas_log(src: str) -> str:
    return os.path.join(CSRC, src.replace(".cu", ".ptxas.txt"))


def resource_report(src: str) -> dict:
    """{mangled kernel name: {"registers", "spill_stores", "spill_loads", "stack"}} from ptxas's own
    report for one source file (written by `build`; compiled again here, without an object file, when
    the library was built by an older copy of this script).  A few extra live values in a softmax loop
    can turn into spills that cost a kernel 15 % without failing any test, so the tests hold the hot
    kernels to a budget."""
    import re
    log = _ptxas_log(src)
    if not os.path.exists(log) or os.path.getmtime(log) < os.path.getmtime(os.path.join(CSRC, src)):
        cmd = [_nvcc(), "-Xptxas=-v", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", os.devnull]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout.decode()}")
        with open(log, "w") as f:
            f.write(r.stdout.decode())
    report, name = {}, None
    for line in open(log):
        m = re.search(r"Compiling entry function '([^']+)'", line)
        if m:
            name = m.group(1)
            report[name] = {"registers": 0, "spill_stores": 0, "spill_loads": 0, "stack": 0}
            continue
        if name is None:
            continue
        m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m:
            report[name].update(stack=int(m.group(1)), spill_stores=int(m.group(2)), spill_loads=int(m.group(3)))
        m = re.search(r"Used (\d+) registers", line)
        if m:
            report[name]["registers"] = int(m.group(1))
    return report


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

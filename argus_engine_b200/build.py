"""Ahead-of-time build of libargus_b200.so for sm_100a (nvcc cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libargus_b200.so")
SOURCES = ["context.cu", "context_kivi.cu", "decode_f16.cu", "decode_kivi.cu", "kivi_ops.cu", "score_reduce.cu", "prefill_sm100.cu", "decode_f16_static.cu", "lse_merge.cu", "kv_cast.cu", "exchange_merge.cu", "kv_ops.cu", "context_kv.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


OUT_STAMPED = os.path.join(HERE, "libargus_b200_stamped.so")


def _stale(out: str = OUT) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "argus_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, stamped: bool = False) -> str:
    """Compile every CUDA source into one shared library beside this file. Returns its path.

    stamped=True builds the diagnostic twin libargus_b200_stamped.so (-DARGUS_XC_PROFILE: the sharded decode's exchange
    tail records globaltimer stamps that `python -m argus_engine_b200.exchange_stamps` prints); never the default."""
    out_path = OUT_STAMPED if stamped else OUT
    if not force and not _stale(out_path):
        return out_path
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".stamped.o" if stamped else ".o"))
        cmd = ["nvcc", *NVCC_FLAGS, *(["-DARGUS_XC_PROFILE"] if stamped else []), "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {src} ---\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call(["nvcc", "-shared", "-o", out_path, *objs, "-Xcompiler", "-fPIC"])
    return out_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, stamped="--stamped" in sys.argv))

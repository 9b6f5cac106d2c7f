"""Build the C-ABI CUDA libraries in-tree (krasis_b200/_lib/) for sm_100a.

Two targets, so that a model only compiles what it runs on:
  "core"  libkrasis_b200.so       MoE prefill path: grouped / dense tcgen05 GEMMs, Gated DeltaNet, GQA / MLA attention, NCCL glue
  "seq"   libkrasis_b200_seq.so   ragged-batch sequence operators (csrc/seq_ops.cu, seq_mix.cu, seq_rec.cu): norms, generic GEMM, windowed
                                  latent attention with an optional sink, short convolution + gated delta rule (decay per head or per
                                  key channel) with state slots, per-head paged multi-map attention (score cap, sink, pooled blocks
                                  before the window, rotated values), gated and ungated linear units, router and routed experts,
                                  gated linear attention and selective scan with state slots, side-by-side mixers, depth average
nvcc cross-compiles without a GPU.  The .so files are git-ignored; a missing or stale one is rebuilt on demand.
"""
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "_lib")
LIB = os.path.join(LIBDIR, "libkrasis_b200.so")
SEQ_LIB = os.path.join(LIBDIR, "libkrasis_b200_seq.so")
SEQ_SOURCES = ["seq_ops.cu", "seq_mix.cu", "seq_rec.cu"]
SOURCES = ["grouped_gemm.cu", "router_gemm.cu", "dense_gemm.cu", "gdn.cu", "gdn_tc.cu", "gqa.cu", "elementwise.cu", "moe_kernels.cu", "capi.cu", "capi_attn.cu", "capi_comm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-Xptxas", "-v",
]


def _stamp(sources=None, header="krasis_b200.h"):
    h = hashlib.sha256()
    for root, _, files in sorted(os.walk(CSRC)):
        for f in sorted(files):
            if sources is None and f in SEQ_SOURCES:
                continue                      # the core library does not depend on the sequence operators
            if sources is not None and f not in sources and not (f.endswith(".cuh") and f.startswith("seq_")):
                continue
            h.update(open(os.path.join(root, f), "rb").read())
    h.update(open(os.path.join(HERE, "..", "include", header), "rb").read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_seq(force: bool = False, verbose: bool = False) -> str:
    """The sequence-operator library alone (one translation unit, well under a minute)."""
    return _build(SEQ_LIB, SEQ_SOURCES, _stamp(SEQ_SOURCES, "krasis_b200_seq.h"), force, verbose)


def build(force: bool = False, verbose: bool = False) -> str:
    return _build(LIB, SOURCES, _stamp(), force, verbose)


def _build(LIB: str, SOURCES, stamp: str, force: bool, verbose: bool) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    stamp_file = LIB + ".stamp"
    if not force and os.path.exists(LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs, procs = [], []
    for src in SOURCES:                       # the translation units compile side by side
        obj = os.path.join(LIBDIR, src.replace(".cu", ".o"))
        cmd = [nvcc, "-c", os.path.join(CSRC, src), "-o", obj] + NVCC_FLAGS
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    failed = []
    for src, obj, proc in procs:
        out, err = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out + err)
        if proc.returncode:
            failed.append(src)
            continue
        with open(obj + ".ptxas.txt", "w") as f:
            f.write(err)
        objs.append(obj)
    if failed:
        raise RuntimeError(f"nvcc failed on {', '.join(failed)}")
    tmp_lib = LIB + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp_lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    os.replace(tmp_lib, LIB)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return LIB


if __name__ == "__main__":
    if "--seq-only" not in sys.argv:
        print(build(force="--force" in sys.argv, verbose=True))
    print(build_seq(force="--force" in sys.argv, verbose=True))

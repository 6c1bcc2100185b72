"""Reference arm of the benchmark: the reference's own native decode kernels, unmodified, on the host CPU.

The reference is a Java 25 / Maven project and cannot be built without a JDK, Maven and the network. Its production decode
GEMM is C: ``gemm_q8_q4`` (``native/src/main/c/simd/vector_simd.c:595``, int8-block activations x JQ4 weights), called once
per projection and token through Panama with the output rows split over a thread pool
(``native/src/main/java/.../NativeSimdTensorOperations.java:223``). That file builds with gcc alone.

``install()`` copies the untouched ``vector_simd.c`` / ``vector_simd.h`` under ``baseline/_ref/native_simd``; ``run()`` compiles
them there for the CPU it runs on (flags of ``native/pom.xml:204``) and times the per-token projection list of the benchmark shape
(q|k|v, o, gate|up, down for every layer, then the JQ4 output head), activations quantised to Q8 blocks the way the reference does
(block 32, scale = max|v| / 127), all host cores. Attention, norms, sampling and the JVM are left out, so the figure is an UPPER
bound of what the reference reaches on this host. The reference has no request batching: concurrent requests are independent
single-token forwards that share the cores, so the aggregate rate is the single-stream rate.
"""
from __future__ import annotations

import ctypes
import json
import os
import shutil
import subprocess
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF_DIR = os.path.join(_ROOT, "baseline", "_ref", "native_simd")
FILES = ("vector_simd.c", "vector_simd.h")
HAS_F16C, HAS_AVX2 = 2, 4  # run-time flags of vector_simd.h:13-14 (the second one selects the 512-bit kernels)


def install(reference_root: str) -> str:
    """Copy the reference's SIMD sources, byte for byte, to ``baseline/_ref/native_simd``."""
    src = os.path.join(reference_root, "native", "src", "main", "c", "simd")
    os.makedirs(REF_DIR, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(REF_DIR, f))
    return REF_DIR


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def build(src_dir: str = REF_DIR) -> str:
    """Compile the sources for this machine's CPU; returns the shared object (rebuilt when the CPU flags changed)."""
    c = os.path.join(src_dir, "vector_simd.c")
    if not os.path.exists(c):
        raise FileNotFoundError(f"{c}: run `python -m deliverance_b200.bench.reference_arm --install <reference checkout>` first")
    tag = "avx512" if "avx512f" in _cpu_flags() else "avx2"
    so = os.path.join(src_dir, f"libdeliverance_ref_{tag}.so")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(c):
        cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-march=native", "-Wno-attributes", "-fPIC", "-fno-omit-frame-pointer", "-shared", c, "-lm", "-o", so]
        subprocess.run(cmd, check=True, capture_output=True, text=True)
    return so


def load(src_dir: str = REF_DIR) -> ctypes.CDLL:
    lib = ctypes.CDLL(build(src_dir))
    vp, i = ctypes.c_void_p, ctypes.c_int
    lib.gemm_q8_q4.argtypes = [i, vp, vp, i, vp, vp, i, vp, i, i, i, i, i, i, i, i, i, i]
    lib.gemm_q8_q4.restype = None
    lib.gemm_f32_q4.argtypes = [i, vp, i, vp, vp, i, vp, i, i, i, i, i, i, i, i, i]
    lib.gemm_f32_q4.restype = None
    return lib


def runtime_flags() -> int:
    return HAS_F16C | (HAS_AVX2 if "avx512f" in _cpu_flags() else 0)


def quantize_q8(x: np.ndarray):
    """Q8 activation blocks as the reference builds them (``tensor/.../Q8ByteBufferTensor.java:57-79``): block 32, scale = max|v| / 127."""
    m, k = x.shape
    b = x.reshape(m, k // 32, 32)
    amax = np.abs(b).max(-1)
    scale = (amax / 127.0).astype(np.float32)
    inv = np.where(amax > 0, 127.0 / np.maximum(amax, 1e-30), 0.0).astype(np.float32)
    q = np.rint(b * inv[..., None]).astype(np.int8).reshape(m, k)
    return q, scale


def projection_list(shape: dict) -> list:
    """(rows, cols, calls per token) of the projections one decoded token passes through."""
    h, L = shape["hidden_size"], shape["num_hidden_layers"]
    d = shape.get("head_dim") or h // shape["num_attention_heads"]
    q, kv = shape["num_attention_heads"] * d, shape["num_key_value_heads"] * d
    inter = shape["intermediate_size"]
    return [(q + 2 * kv, h, L), (h, q, L), (2 * inter, h, L), (h, inter, L), (shape["vocab_size"], h, 1)]


def run(args, shape: dict, threads: int | None = None) -> dict:
    lib = load()
    flags = runtime_flags()
    threads = threads or os.cpu_count() or 1
    rng = np.random.default_rng(0)
    pool = ThreadPoolExecutor(threads)
    mats = []
    for (n, k, calls) in projection_list(shape):
        # random packed nibbles and scales: the kernel's time does not depend on the values
        mats.append((n, k, calls, rng.integers(0, 256, (n, k // 2), dtype=np.uint8), (rng.random((n, k // 32), dtype=np.float32) * 0.01 + 1e-3)))
    acts = {k: quantize_q8(rng.standard_normal((1, k), dtype=np.float32)) for (_, k, _, _, _) in mats}
    outs = {n: np.zeros((1, n), dtype=np.float32) for (n, _, _, _, _) in mats}

    def one(n, k, b, bf):
        a, af = acts[k]
        r = outs[n]
        per = (n + threads - 1) // threads

        def chunk(t):
            n0 = t * per
            cnt = min(per, n - n0)
            if cnt > 0:  # the reference's thread pool hands each worker a range of output rows (n0, n)
                lib.gemm_q8_q4(flags, af.ctypes.data, a.ctypes.data, 0, bf.ctypes.data, b.ctypes.data, 0, r.ctypes.data, 0, 1, n0, cnt, k, k, k // 32, k // 2, k // 32, n)

        list(pool.map(chunk, range(threads)))

    def token():
        for (n, k, calls, b, bf) in mats:
            for _ in range(calls):
                one(n, k, b, bf)

    for _ in range(max(1, min(args.warmup, 3))):
        token()
    steps = max(1, min(args.steps, 8))  # a token takes seconds on the host; a few are enough for a stable mean
    t0 = time.perf_counter()
    for _ in range(steps):
        token()
    dt = (time.perf_counter() - t0) / steps
    pool.shutdown()
    return {"tok_s": 1.0 / dt, "ms_per_token": dt * 1e3, "threads": threads, "tokens_timed": steps,
            "isa": "avx512" if flags & HAS_AVX2 else "avx2"}


def main() -> int:
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--install", metavar="REFERENCE_ROOT", help="copy vector_simd.c / .h from a reference checkout")
    ap.add_argument("--shape", default="qwen3-4b")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=1)
    a = ap.parse_args()
    if a.install:
        print("installed", install(a.install))
        return 0
    from deliverance_b200.ckpt.synthetic import SHAPES

    print(json.dumps(run(a, SHAPES[a.shape])))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

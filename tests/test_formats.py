"""JQ4 / safetensors / quantiser / shard loader / LoRA: format invariants on the CPU."""
import json
import os
import struct

import pytest
import torch

from deliverance_b200.ckpt.jq4 import q4_dequantize, q4_quantize, q4_scalar_reference, q8_dequantize, q8_quantize
from deliverance_b200.ckpt.loader import ShardSpec, WeightLoader
from deliverance_b200.ckpt.lora import LoraAdapter, MergingWeightLoader, apply_lora_delta, base_name, lora_names
from deliverance_b200.ckpt.quantizer import DEFAULT_Q4_FILTER, FINISHED, MANIFEST, ModelQuantizer, quantize_on_demand
from deliverance_b200.ckpt.safetensors_io import Q4Tensor, SafeTensorFile, write_safetensors, write_sharded
from deliverance_b200.ckpt.tiny import write_tiny_model


def test_q4_matches_scalar_definition():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(8, 64, generator=g)
    w[1, :32] = 0.0
    w[2, 5] = 9.0
    w[3, 40] = -9.0
    packed, scales = q4_quantize(w)
    assert packed.shape == (8, 32) and scales.shape == (8, 2)
    for r in range(8):
        for b in range(2):
            ref_bytes, ref_scale = q4_scalar_reference(w[r, b * 32 : (b + 1) * 32].tolist())
            assert bytes(packed[r, b * 16 : (b + 1) * 16].tolist()) == ref_bytes
            assert struct.pack("<f", scales[r, b].item()) == struct.pack("<f", ref_scale)


def test_q4_layout_and_roundtrip():
    w = torch.zeros(1, 32)
    w[0, 0] = -8.0  # largest magnitude -> nibble 0 ... scale = -8 / -8 = 1
    w[0, 16] = 7.0
    w[0, 1] = 1.0
    packed, scales = q4_quantize(w)
    assert scales[0, 0].item() == 1.0
    assert packed[0, 0].item() == (0 | (15 << 4))  # byte j = q[j] | q[j+16] << 4
    assert packed[0, 1].item() == (9 | (8 << 4))
    d = q4_dequantize(packed, scales)
    assert d[0, 0].item() == -8.0 and d[0, 16].item() == 7.0 and d[0, 1].item() == 1.0
    g = torch.Generator().manual_seed(1)
    x = torch.randn(16, 128, generator=g)
    p, s = q4_quantize(x)
    err = (q4_dequantize(p, s) - x).abs().max() / x.abs().max()
    assert err < 0.15
    with pytest.raises(ValueError):
        q4_quantize(torch.randn(2, 30))


def test_q8_roundtrip():
    x = torch.randn(4, 64)
    q, s = q8_quantize(x)
    assert q.dtype == torch.int8 and s.shape == (4, 2)
    assert (q8_dequantize(q, s) - x).abs().max() < x.abs().max() / 100


def test_loader_dequantises_i8_block_weights(tmp_path):
    """An ``I8`` entry with a ``.qb`` scale sidecar (block-32 int8 weights) loads as a dense tensor; a plain int8 tensor stays."""
    from deliverance_b200.ckpt.loader import WeightLoader

    x = torch.randn(4, 64)
    q, s = q8_quantize(x)
    write_safetensors(str(tmp_path / "model.safetensors"), {"w.weight": q, "w.weight.qb": s, "plain": torch.arange(4, dtype=torch.int8)})
    ld = WeightLoader(str(tmp_path))
    w = ld.load("w.weight")
    assert w.dtype == torch.bfloat16 and (w.float() - x).abs().max() < x.abs().max() / 50
    assert ld.load("plain").dtype == torch.int8 and "w.weight.qb" not in ld.names()


def test_safetensors_roundtrip_with_q4(tmp_path):
    w = torch.randn(4, 64)
    p, s = q4_quantize(w)
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, {"a.weight": Q4Tensor(p, s, (4, 64)), "b": torch.arange(6, dtype=torch.int32).reshape(2, 3),
                             "c": torch.randn(5).to(torch.bfloat16)}, metadata={"format": "pt"})
    f = SafeTensorFile(path)
    assert f.infos["a.weight"].dtype == "Q4" and f.infos["a.weight"].shape == (4, 64) and f.infos["a.weight"].nbytes == 128
    assert f.infos["a.weight.qb"].dtype == "F32" and f.infos["a.weight.qb"].shape == (4, 2)
    assert torch.equal(f.tensor("a.weight"), p) and torch.equal(f.tensor("b"), torch.arange(6, dtype=torch.int32).reshape(2, 3))
    assert f.metadata == {"format": "pt"}
    with open(path, "rb") as fh:
        (hlen,) = struct.unpack("<Q", fh.read(8))
        json.loads(fh.read(hlen))
    # the standard safetensors reader sees the dense entries
    from safetensors import safe_open
    with pytest.raises(Exception):
        with safe_open(path, "pt") as sf:
            sf.get_tensor("a.weight")  # non-standard dtype


def test_sharded_index_and_loader(tmp_path):
    d = str(tmp_path / "m")
    tensors = {f"t{i}": torch.randn(64, 64) for i in range(6)}
    files = write_sharded(d, tensors, max_shard_bytes=40_000)
    assert len(files) > 1 and os.path.exists(os.path.join(d, "model.safetensors.index.json"))
    wl = WeightLoader(d)
    assert sorted(wl.names()) == sorted(tensors)
    for k, v in tensors.items():
        assert torch.equal(wl.load(k), v)
    assert wl.majority_dtype() == "F32"


def test_shards_row_col_q4_alignment(tmp_path):
    w = torch.randn(8, 128)
    p, s = q4_quantize(w)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {"w": Q4Tensor(p, s, (8, 128)), "d": w})
    wl = WeightLoader(str(tmp_path))
    full = wl.load("w").dequantize()
    r1 = wl.load("w", ShardSpec("row", 1, 2)).dequantize()
    assert torch.equal(r1, full[4:])
    c0 = wl.load("w", ShardSpec("col", 0, 2)).dequantize()
    assert torch.equal(c0, full[:, :64])
    assert torch.equal(wl.load("d", ShardSpec("col", 1, 4)), w[:, 32:64])
    g = wl.load("d", ShardSpec("row", 1, 2, groups=2))  # fused gate|up style: each half split
    assert torch.equal(g, torch.cat([w[2:4], w[6:8]]))
    with pytest.raises(ValueError):
        wl.load("w", ShardSpec("col", 0, 8))  # 16-column shards break the 32-element blocks
    assert wl.majority_dtype() in ("Q4", "F32")


def test_default_filter():
    yes = ["model.layers.0.self_attn.q_proj.weight", "model.layers.3.mlp.down_proj.weight", "model.layers.1.mlp.experts.7.up_proj.weight",
           "model.layers.0.block_sparse_moe.experts.1.w2.weight", "bert.encoder.layer.0.attention.self.query.weight",
           "model.layers.0.mamba.in_proj.weight", "model.layers.0.shared_mlp.input_linear.weight"]
    no = ["model.embed_tokens.weight", "lm_head.weight", "model.norm.weight", "model.layers.0.mlp.gate.weight",
          "model.layers.0.self_attn.q_proj.weight.qb", "model.layers.0.self_attn.q_proj.bias", "model.layers.0.block_sparse_moe.gate.weight"]
    assert all(DEFAULT_Q4_FILTER(n) for n in yes) and not any(DEFAULT_Q4_FILTER(n) for n in no)


def test_model_quantizer_and_on_demand(tmp_path):
    src = str(tmp_path / "src")
    write_tiny_model(src, "llama", seed=0)
    out = str(tmp_path / "out")
    man = ModelQuantizer().quantize(src, out)
    assert os.path.exists(os.path.join(out, FINISHED)) and os.path.exists(os.path.join(out, MANIFEST))
    assert os.path.exists(os.path.join(out, "config.json"))
    wl = WeightLoader(out)
    assert wl.is_q4("model.layers.0.self_attn.q_proj.weight") and not wl.is_q4("model.embed_tokens.weight")
    assert wl.info("model.norm.weight").shape == (1, 64)  # 1-D tensors are rewritten as [1, N]
    assert len(man["tensors"]) == 2 * 7
    src_w = WeightLoader(src).load("model.layers.0.mlp.up_proj.weight")
    p, s = q4_quantize(src_w)
    q = wl.load("model.layers.0.mlp.up_proj.weight")
    assert torch.equal(q.packed, p) and torch.equal(q.scales, s)
    target = str(tmp_path / "cache" / "m-JQ4")
    os.makedirs(os.path.dirname(target))
    assert quantize_on_demand(src, target) == target
    stamp = os.path.getmtime(os.path.join(target, FINISHED))
    assert quantize_on_demand(src, target) == target and os.path.getmtime(os.path.join(target, FINISHED)) == stamp


def _write_adapter(path, base_shape, r=4, alpha=8.0, name="model.layers.0.self_attn.q_proj.weight"):
    os.makedirs(path, exist_ok=True)
    A, B = torch.randn(r, base_shape[1]) * 0.1, torch.randn(base_shape[0], r) * 0.1
    a_name, b_name = lora_names(name)
    write_safetensors(os.path.join(path, "adapter_model.safetensors"), {a_name: A, b_name: B})
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": ["q_proj"], "peft_type": "LORA"}, f)
    return A, B


def test_lora_names_merge_and_delta(tmp_path):
    n = "model.layers.0.self_attn.q_proj.weight"
    a, b = lora_names(n)
    assert a == "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" and base_name(a) == n and base_name(b) == n
    src = str(tmp_path / "src")
    write_tiny_model(src, "llama", seed=0)
    base = WeightLoader(src).load(n).clone()
    A, B = _write_adapter(str(tmp_path / "ad"), base.shape)
    ad = LoraAdapter(str(tmp_path / "ad"))
    assert ad.targets() == [n] and ad.config.scale == 2.0
    merged = MergingWeightLoader(src, ad).load(n)
    assert torch.allclose(merged, base + 2.0 * (B @ A), atol=1e-6)
    with pytest.raises(ValueError):
        MergingWeightLoader(src, ad).load(n, ShardSpec("row", 0, 2))
    x = torch.randn(3, base.shape[1])
    Ar, Bs = ad.resolved(n)
    y = apply_lora_delta(x, x @ base.t(), Ar, Bs)
    assert torch.allclose(y, x @ merged.t(), atol=1e-5)


def test_jq4_properties_hypothesis():
    """Property tests: the quantiser never errs by more than one step of its block, nibble 0 sits on the block's largest
    magnitude, tile packing for the tensor-core GEMM is lossless for ragged shapes, and row interleaving commutes with packing."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    from deliverance_b200 import ops
    from deliverance_b200.ckpt.jq4 import q4_dequantize

    @settings(max_examples=40, deadline=None)
    @given(st.integers(1, 5), st.integers(1, 6), st.integers(0, 2**31 - 1), st.floats(1e-3, 50.0))
    def quant(rows, blocks, seed, spread):
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(rows, blocks * 32, generator=g) * spread
        p, s = q4_quantize(w)
        err = (q4_dequantize(p, s) - w).abs().reshape(rows, blocks, 32)
        step = s.abs().reshape(rows, blocks, 1)
        assert bool((err <= step * 1.0 + 1e-5 * spread).all())  # half a step from rounding, up to one where nibble 15 clamps
        blk = w.reshape(rows, blocks, 32)
        amax = blk.abs().argmax(dim=2, keepdim=True)
        deq = q4_dequantize(p, s).reshape(rows, blocks, 32)
        assert torch.allclose(deq.gather(2, amax), blk.gather(2, amax), rtol=1e-5, atol=1e-6 * spread)  # the extreme is exact (nibble 0 = -8)

    @settings(max_examples=25, deadline=None)
    @given(st.integers(1, 300), st.integers(1, 9), st.integers(0, 2**31 - 1))
    def tiles(n, kblocks, seed):
        g = torch.Generator().manual_seed(seed)
        k = kblocks * 32
        packed = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
        scales = torch.randn(n, k // 32, generator=g)
        t = ops.prepack_q4(packed, scales)
        assert t.shape == ((n + 127) // 128, (k + 127) // 128, 10240)
        p2, s2 = ops.unpack_q4(t, n, k)
        assert torch.equal(p2, packed) and torch.equal(s2, scales)

    quant()
    tiles()
    g = torch.Generator().manual_seed(1)
    pg, sg = q4_quantize(torch.randn(128, 64, generator=g))
    pu, su = q4_quantize(torch.randn(128, 64, generator=g))
    mixed = ops.interleave_gate_up(Q4Tensor(pg, sg, (128, 64)), Q4Tensor(pu, su, (128, 64)))
    assert torch.equal(mixed.packed[64:128], pu[:64]) and torch.equal(mixed.scales[128:192], sg[64:128]) and mixed.shape == (256, 64)


def _reference_simd():
    """The reference's own C kernels, compiled from an unmodified copy: from ``DLV_REFERENCE_ROOT`` (a checkout of the reference) when
    set, else from the copy the benchmark's reference arm installed under ``baseline/_ref``; None when neither is there or gcc is missing."""
    import shutil
    import subprocess
    import tempfile

    from deliverance_b200.bench import reference_arm as ra

    if shutil.which("gcc") is None:
        return None
    root = os.environ.get("DLV_REFERENCE_ROOT")
    try:
        if root:
            src = os.path.join(root, "native", "src", "main", "c", "simd")
            if not os.path.exists(os.path.join(src, "vector_simd.c")):
                return None
            tmp = tempfile.mkdtemp(prefix="dlv_ref_simd_")
            for f in ra.FILES:
                shutil.copyfile(os.path.join(src, f), os.path.join(tmp, f))
            return ra.load(tmp)
        if not os.path.exists(os.path.join(ra.REF_DIR, "vector_simd.c")):
            return None
        return ra.load()
    except (OSError, subprocess.CalledProcessError):
        return None


def test_jq4_blocks_against_the_reference_c_kernel():
    """JQ4 packing pinned by an oracle this repo did not write: the reference's ``gemm_f32_q4`` (native/src/main/c/simd/vector_simd.c:1145,
    scalar walk of the packed nibbles and block scales) multiplies the identity by weights packed with ``q4_quantize``; the product must
    be the transpose of ``q4_dequantize`` to rounding."""
    lib = _reference_simd()
    if lib is None:
        pytest.skip("no reference C sources (set DLV_REFERENCE_ROOT or install the benchmark's reference arm) or no gcc")
    import numpy as np

    g = torch.Generator().manual_seed(11)
    n, k = 48, 256
    w = torch.randn(n, k, generator=g) * 0.3
    w[5, 32:64] = 0.0      # an all-zero block
    w[7, 3] = -4.0         # the block maximum is negative
    packed, scales = q4_quantize(w)
    deq = q4_dequantize(packed, scales).numpy()
    a = np.eye(k, dtype=np.float32)
    p_np = np.ascontiguousarray(packed.numpy())
    s_np = np.ascontiguousarray(scales.numpy().astype(np.float32))
    r = np.zeros((k, n), dtype=np.float32)
    lib.gemm_f32_q4(0, a.ctypes.data, 0, s_np.ctypes.data, p_np.ctypes.data, 0, r.ctypes.data, 0, k, 0, n, k, k, k // 2, k // 32, n)
    assert np.abs(r.T - deq).max() <= 1e-6
    # and a real product, against the dequantised weights in fp32
    x = torch.randn(5, k, generator=g).numpy().astype(np.float32)
    r2 = np.zeros((5, n), dtype=np.float32)
    lib.gemm_f32_q4(0, x.ctypes.data, 0, s_np.ctypes.data, p_np.ctypes.data, 0, r2.ctypes.data, 0, 5, 0, n, k, k, k // 2, k // 32, n)
    assert np.abs(r2 - x @ deq.T).max() <= 1e-4


def test_quantizer_command_line_then_generate(tmp_path):
    """``python -m deliverance_b200.ckpt.quantizer SRC OUT`` as a user runs it; the quantised directory then loads through the public
    builder and generates, like the source directory does."""
    import subprocess
    import sys

    from deliverance_b200.api import AutoModelForCausalLM
    from deliverance_b200.params import GeneratorParameters

    src, out = str(tmp_path / "src"), str(tmp_path / "jq4")
    write_tiny_model(src, "llama", seed=4, std=0.05)
    r = subprocess.run([sys.executable, "-m", "deliverance_b200.ckpt.quantizer", src, out], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "quantised" in r.stdout, r.stderr[-500:]
    assert os.path.exists(os.path.join(out, FINISHED))
    clm_q = AutoModelForCausalLM.new_builder(out).with_device("cpu").build()
    clm_f = AutoModelForCausalLM.new_builder(src).with_device("cpu").build()
    p = GeneratorParameters(max_tokens=8, temperature=0.0)
    ids = [5, 9, 33, 17, 4]
    a, b = clm_q.generate(ids, p), clm_f.generate(ids, p)
    assert len(a.token_ids) == 8 and len(b.token_ids) == 8 and a.generated_tokens == 8
    assert WeightLoader(out).is_q4("model.layers.0.mlp.down_proj.weight")

#!/usr/bin/env python3
"""Generate tests/golden/*.npz from the reference's own Python restatement.

Run in a container that has the reference checkout and the `gguf` package:

    python tests/golden/make_golden.py /path/to/reference      (or MNEMO_REFERENCE_DIR=...)

It imports tools/validate_dequant.py from the reference (its functions, not
its main(), which needs a private model file) and gguf.quants, feeds them
seeded and hand-built blocks, and stores inputs + outputs. Tests then check
the C oracle against these files with ==, so the oracle is pinned to the
reference's dequant semantics without the reference being present.

Vectors:
  q4k_seeded / q6k_seeded : random blocks from mnemocuda_b200.synth
  q4k_known  / q6k_known  : hand-built blocks (all zero, all 0xFF, one hot
                            nibble, subnormal and negative d, max scales)
  ragged                  : n_cols not a multiple of 256
  scale_min               : get_scale_min_k4 on every j for random 12-byte rows
  q5k_* / q8_0_*          : seeded and ragged blocks through dequant_q5k_cuda_style / dequant_q8_0_cuda_style
                            (the validator has no Q3_K function; that type is checked on the GPU against
                            the reference's compiled kernel instead)
support_golden.npz (from tools/validate_rope_norm.py's kernel replicas):
  rms_*                   : kernel_rms_norm on seeded vectors (hidden 2048 / 4096, head 128)
  rope_*                  : kernel_rope at positions 0, 1, 17, 4095, 8191 (16 + 2 heads of 128)
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))
from mnemocuda_b200 import synth  # noqa: E402


def load_reference(ref_root: str, name: str = "validate_dequant"):
    path = os.path.join(ref_root, "tools", name + ".py")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def support_vectors(ref_root: str) -> dict:
    """RMSNorm and RoPE: outputs of the reference's own numpy replicas of its kernels."""
    vr = load_reference(ref_root, "validate_rope_norm")
    out = {}
    for tag, n, seed in (("h2048", 2048, 31), ("h4096", 4096, 32), ("head128", 128, 33)):
        x = synth.normal_f32(seed, n, 3.0)
        w = (1.0 + 0.1 * synth.normal_f32(seed + 100, n)).astype(np.float32)
        out[f"rms_{tag}_x"], out[f"rms_{tag}_w"] = x, w
        out[f"rms_{tag}_ref"] = np.asarray(vr.kernel_rms_norm(x.astype(np.float64), w.astype(np.float64), 1e-6), np.float64)
    nh, hd, theta = 18, 128, 1_000_000.0
    vec = synth.normal_f32(41, nh * hd)
    out["rope_in"] = vec
    out["rope_pos"] = np.array([0, 1, 17, 4095, 8191], np.int32)
    out["rope_ref"] = np.stack([np.asarray(vr.kernel_rope(vec.astype(np.float64), nh, hd, int(p), theta), np.float64)
                                for p in out["rope_pos"]])
    out["rope_meta"] = np.array([nh, hd, theta], np.float64)
    return out


def known_q4k() -> np.ndarray:
    f16 = lambda v: np.array([v], np.float16).view(np.uint8)
    blocks = []
    b = np.zeros(144, np.uint8)                       # all zero
    blocks.append(b.copy())
    b[:] = 0xFF                                       # all ones: d = dmin = NaN pattern avoided below
    b[0:2] = f16(1.0); b[2:4] = f16(1.0)
    blocks.append(b.copy())
    b = np.zeros(144, np.uint8)                       # single hot nibble, weight 0
    b[0:2] = f16(0.5); b[2:4] = f16(0.25); b[4:16] = 0x21; b[16] = 0x0F
    blocks.append(b.copy())
    b = np.zeros(144, np.uint8)                       # single hot high nibble, weight 255
    b[0:2] = f16(2.0); b[2:4] = f16(0.0); b[4:16] = 0xFF; b[143] = 0xF0
    blocks.append(b.copy())
    b = synth.q4k_blocks(77, 1)[0]                    # subnormal d, negative dmin
    b[0:2] = np.array([0x0003], np.uint16).view(np.uint8)
    b[2:4] = f16(-1.5e-3)
    blocks.append(b.copy())
    b = synth.q4k_blocks(78, 1)[0]                    # smallest normal / largest subnormal
    b[0:2] = np.array([0x0400], np.uint16).view(np.uint8)
    b[2:4] = np.array([0x03FF], np.uint16).view(np.uint8)
    blocks.append(b.copy())
    b = synth.q4k_blocks(79, 1)[0]                    # scales with every high-bit combination
    b[4:16] = np.array([0xC0, 0x80, 0x40, 0x3F, 0xFF, 0x7F, 0xBF, 0x00, 0xF0, 0x0F, 0xA5, 0x5A], np.uint8)
    blocks.append(b.copy())
    return np.stack(blocks)


def known_q6k() -> np.ndarray:
    f16 = lambda v: np.array([v], np.float16).view(np.uint8)
    blocks = []
    b = np.zeros(210, np.uint8)
    blocks.append(b.copy())                           # all zero (q = -32, scale 0)
    b = np.zeros(210, np.uint8); b[192:208] = 1; b[208:210] = f16(1.0)
    blocks.append(b.copy())                           # q = -32 everywhere
    b = np.full(210, 0xFF, np.uint8); b[192:208] = 0x7F; b[208:210] = f16(1.0)
    blocks.append(b.copy())                           # q = +31, scale +127
    b = np.zeros(210, np.uint8); b[192:208] = 0x80; b[208:210] = f16(-2.0)
    b[5] = 0x3C; b[128 + 5] = 0b10011100
    blocks.append(b.copy())                           # scale -128, negative d, one hot position
    b = synth.q6k_blocks(81, 1)[0]
    b[208:210] = np.array([0x0001], np.uint16).view(np.uint8)  # smallest subnormal d
    blocks.append(b.copy())
    b = synth.q6k_blocks(82, 1)[0]
    b[192:208] = np.arange(-8, 8, dtype=np.int8).view(np.uint8)
    blocks.append(b.copy())
    return np.stack(blocks)


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MNEMO_REFERENCE_DIR", "")
    if not ref_root or not os.path.isdir(ref_root):
        sys.exit("usage: make_golden.py /path/to/reference (or set MNEMO_REFERENCE_DIR)")
    vd = load_reference(ref_root)
    from gguf import dequantize
    from gguf.quants import GGMLQuantizationType as T

    out = {}

    # --- Q4_K seeded: 3 rows x 1024 columns (12 blocks) --------------------
    w = synth.q4k_matrix(11, 3, 1024)
    out["q4k_seeded_w"] = w
    out["q4k_seeded_ref"] = vd.dequant_q4k_cuda_style(w.tobytes(), 3, 1024)
    g = dequantize(w.reshape(3, -1), T.Q4_K)
    assert np.array_equal(g, out["q4k_seeded_ref"]), "reference validator != gguf (Q4_K)"

    # --- Q6_K seeded -------------------------------------------------------
    w = synth.q6k_matrix(12, 3, 1024)
    out["q6k_seeded_w"] = w
    out["q6k_seeded_ref"] = vd.dequant_q6k_reference(w.tobytes(), 3, 1024)
    g = dequantize(w.reshape(3, -1), T.Q6_K)
    assert np.array_equal(g, out["q6k_seeded_ref"]), "reference validator != gguf (Q6_K)"

    # --- hand-built blocks (one row each, 256 columns) ---------------------
    k4 = known_q4k()
    out["q4k_known_w"] = k4
    out["q4k_known_ref"] = vd.dequant_q4k_cuda_style(k4.tobytes(), k4.shape[0], 256)
    assert np.array_equal(dequantize(k4, T.Q4_K), out["q4k_known_ref"], equal_nan=True)
    k6 = known_q6k()
    out["q6k_known_w"] = k6
    out["q6k_known_ref"] = vd.dequant_q6k_reference(k6.tobytes(), k6.shape[0], 256)
    assert np.array_equal(dequantize(k6, T.Q6_K), out["q6k_known_ref"], equal_nan=True)

    # --- ragged widths: 2 rows, n_cols = 300 (2 blocks per row, 2nd partial) -
    w = synth.q4k_matrix(13, 2, 300)
    out["q4k_ragged_w"] = w
    out["q4k_ragged_ref"] = vd.dequant_q4k_cuda_style(w.tobytes(), 2, 300)
    w = synth.q6k_matrix(14, 2, 300)
    out["q6k_ragged_w"] = w
    out["q6k_ragged_ref"] = vd.dequant_q6k_reference(w.tobytes(), 2, 300)

    # --- Q5_K and Q8_0 (the validator's restatements of the reference kernels) ---
    for tag, tid, fn, gt in (("q5k", 13, vd.dequant_q5k_cuda_style, None), ("q8_0", 8, vd.dequant_q8_0_cuda_style, T.Q8_0)):
        for name, seed, rows, cols in (("seeded", 16, 3, 1024), ("ragged", 17, 2, 300)):
            w = synth.typed_matrix(tid, seed, rows, cols)
            out[f"{tag}_{name}_w"] = w
            out[f"{tag}_{name}_ref"] = np.asarray(fn(w.tobytes(), rows, cols), np.float32)
            if gt is not None and name == "seeded":
                assert np.array_equal(dequantize(w.reshape(rows, -1), gt), out[f"{tag}_{name}_ref"])

    # --- get_scale_min_k4 --------------------------------------------------
    sc_in = synth.words(15, 0, 48).view(np.uint8).reshape(32, 12)
    sc_out = np.zeros((32, 8, 2), np.uint8)
    for r in range(32):
        for j in range(8):
            sc_out[r, j] = vd.get_scale_min_k4(j, [int(v) for v in sc_in[r]])
    out["scale_min_in"] = sc_in
    out["scale_min_out"] = sc_out

    # --- f16 -> f32 over every bit pattern (validator's f16_to_f32 == numpy) --
    allh = np.arange(65536, dtype=np.uint16)
    probe = [0, 1, 0x3FF, 0x400, 0x3C00, 0x7BFF, 0x8001, 0xBC00, 0xFBFF]
    for h in probe:
        assert np.array_equal(vd.f16_to_f32(h), allh[h:h + 1].view(np.float16).astype(np.float32)[0])
    # stored as a checksum only; the test regenerates it with numpy
    out["f16_probe"] = np.array(probe, np.uint16)
    out["f16_probe_ref"] = np.array([vd.f16_to_f32(h) for h in probe], np.float32)

    sup = support_vectors(ref_root)
    np.savez_compressed(os.path.join(HERE, "support_golden.npz"), **sup)
    print("wrote", os.path.join(HERE, "support_golden.npz"), {k: v.shape for k, v in sup.items()})

    np.savez_compressed(os.path.join(HERE, "dequant_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "dequant_golden.npz"),
          {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()

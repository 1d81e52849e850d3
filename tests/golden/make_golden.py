"""Generates the golden fixtures of this folder from the reference itself.  Run on a machine that has
the reference checkout (environment variable EET_REFERENCE):

    make -C oracle ref && python tests/golden/make_golden.py

* quant_*.npz    - inputs and outputs of the reference's symmetric_quantize + packer
                   (3rdparty/cutlass_kernels/cutlass_preprocessors.cc:581-678, :497-534) compiled for the
                   host as oracle/_ref/libeet_ref_quant.so
* alibi.npz      - _get_interleave / _gen_alibi_mask of python/eet/transformers/modeling_baichuan.py:51-80,
                   executed from the reference file's own source text (the module itself cannot be imported:
                   it needs the compiled EET extension)
* names.json     - convert_name (python/eet/utils/mapping.py:298-324) applied to the HF LLaMA / Baichuan
                   parameter names

The fixtures are small (tens of KB) and committed; tests compare the oracle and the CUDA kernels with
them on machines where the reference is absent.
"""
import ast
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import w8  # noqa: E402

REF = os.environ.get("EET_REFERENCE", "/root/reference")


def quant_case(name, w):
    q, packed, scales = w8.ref_symmetric_quantize_int8(w)
    np.savez_compressed(os.path.join(HERE, f"quant_{name}.npz"), w=w, q=q, ref_packed=packed, scales=scales)
    print(name, w.shape, w.dtype, "q range", q.min(), q.max())


def edge_matrix(dtype):
    """64 x 128: every column is one edge case of the quantizer."""
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((64, 128)) * 0.02).astype(np.float32)
    w[:, 0] = 0.0                                   # all-zero column: 0/0 -> NaN -> q = 127, scale = 0
    w[:, 1] = 0.0
    w[3, 1] = 1.0                                   # single non-zero: +amax -> clipped to +127
    w[:, 2] = 0.0
    w[5, 2] = -1.0                                  # -amax -> -128
    w[:, 3] = np.linspace(-1, 1, 64)                # both signs of amax present
    k = np.arange(64)
    w[:, 4] = (k - 32 + 0.5) / 128.0                # exact .5 ties at scale 1/128 * amax
    w[0, 4] = 1.0
    w[:, 5] = 6.0e-8                                # denormal fp16 range
    w[:, 6] = 65504.0                               # fp16 max
    w[7, 7] = np.nan                                # NaN element: ignored by amax, quantizes to 127
    w[:, 8] = np.inf                                # inf column: scale inf, q = 127 (inf/inf = NaN)
    w[:, 9] = 0.0
    w[9, 9] = -np.inf
    w[:, 10] = 1e-3 * (k % 7 - 3)
    w[:, 11] = -w[:, 10]
    return w.astype(dtype)


def main():
    assert w8.ref_lib() is not None, "build oracle/_ref first: make -C oracle ref"
    rng = np.random.default_rng(0)
    quant_case("fp16_128x192", (rng.standard_normal((128, 192)) * 0.02).astype(np.float16))
    quant_case("fp32_64x128", (rng.standard_normal((64, 128)) * 0.02).astype(np.float32))
    quant_case("fp16_192x64_wide", (rng.standard_normal((192, 64)) * 3.0).astype(np.float16))
    with np.errstate(all="ignore"):
        quant_case("fp16_edges", edge_matrix(np.float16))
        quant_case("fp32_edges", edge_matrix(np.float32))

    src = open(os.path.join(REF, "python/eet/transformers/modeling_baichuan.py")).read()
    ns = {"math": math, "torch": torch}
    for node in ast.parse(src).body:
        if isinstance(node, ast.FunctionDef) and node.name in ("_get_interleave", "_fill_with_neg_inf", "_gen_alibi_mask"):
            exec(compile(ast.Module([node], []), "modeling_baichuan.py", "exec"), ns)
    np.savez_compressed(os.path.join(HERE, "alibi.npz"),
                        slopes_40=np.array(ns["_get_interleave"](40), dtype=np.float64),
                        slopes_32=np.array(ns["_get_interleave"](32), dtype=np.float64),
                        mask_40x12=ns["_gen_alibi_mask"](40, 12).numpy(),
                        mask_8x33_fp16=ns["_gen_alibi_mask"](8, 33).half().numpy())

    src = open(os.path.join(REF, "python/eet/utils/mapping.py")).read()
    ns = {}
    exec(compile(src, "mapping.py", "exec"), ns)
    names = {}
    for model, keys in (("llama", ["layers.3.self_attn.qkv_proj.weight", "layers.3.self_attn.o_proj.weight",
                                   "layers.0.input_layernorm.weight", "layers.11.mlp.gate_proj.weight",
                                   "layers.11.mlp.up_proj.weight", "layers.11.mlp.down_proj.weight",
                                   "layers.31.post_attention_layernorm.weight"]),
                        ("baichuan", ["layers.2.self_attn.W_pack.weight", "layers.2.self_attn.o_proj.weight",
                                      "layers.39.mlp.down_proj.weight", "layers.39.input_layernorm.weight"])):
        names[model] = {k: ns["convert_name"](k, model) for k in keys}
    json.dump(names, open(os.path.join(HERE, "names.json"), "w"), indent=1, sort_keys=True)
    print(names)


if __name__ == "__main__":
    main()

"""Golden files of the on-disk side, written by the executing reference.

    python tests/golden/make_format_golden.py OUTPUT_DIR

needs oracle/_ref/libcaif_ref_layers.so (`python oracle/build_ref_layers.py`: the reference's own
translation units, unmodified).  Two outputs:

  weight_mapper.json            a rule set and, for a list of probe names, what the reference's
                                CAIF_WeightMapper answers (HfToAif, AifToHf, MissingNames, UnmappedHfNames,
                                RequiredHfNames).  No device involved.
  reference_written.safetensors a file CAIF_SafeTensorsFormat::Save wrote from seeded tensors (F32, F16, BF16,
                                I8 and an odd-length I4) plus metadata; the tensors go through
                                CAIF_DeviceTensor, so this part needs a GPU and is skipped without one.

tests/test_safetensors.py reads both back through this repository's reader and mapper; `format_cases()` below
is shared with it so that the expected tensor bytes are regenerated, not stored twice.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

RULES = [(0, "model.layers.", "blocks."), (0, "model.", "core."), (0, "model.layers.0.", "first."),
         (0, "lm_head.", "head."), (1, "model.embed_tokens.weight", "embedding.table"),
         (1, "model.norm.weight", "final_norm.gamma")]
HF_PROBES = ["model.layers.3.mlp.up_proj.weight", "model.layers.0.self_attn.q_proj.weight", "model.norm.weight",
             "model.embed_tokens.weight", "lm_head.weight", "model.rotary.inv_freq", "unrelated.tensor", "model.",
             "mode", ""]
AIF_PROBES = ["blocks.3.mlp.up_proj.weight", "first.self_attn.q_proj.weight", "final_norm.gamma", "embedding.table",
              "head.weight", "core.rotary.inv_freq", "nothing.here", "core.", "blocks.", ""]

# CAIF_DataType_e values (include/caif/caif_data_type.h) beside the SafeTensors names
F32, F16, BF16, I4, I8 = 0, 2, 3, 4, 5
NAMES = {F32: "F32", F16: "F16", BF16: "BF16", I4: "I4", I8: "I8"}
METADATA = {"framework": "CAIF", "note": "quote \" backslash \\ tab \t done"}


def format_cases():
    """[(name, dtype code, shape, bytes)] in file order, from a fixed seed."""
    rng = np.random.default_rng(2024)
    w32 = rng.standard_normal((3, 5)).astype(np.float32)
    w16 = rng.standard_normal((4, 2)).astype(np.float16)
    bf = (rng.standard_normal(7).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    q8 = rng.integers(-127, 128, (6, 4)).astype(np.int8)
    q4 = rng.integers(0, 256, 8).astype(np.uint8)      # 15 int4 codes: (15 + 1) / 2 bytes
    q4[-1] &= 0x0F
    scales = rng.uniform(0.001, 0.02, 1).astype(np.float16)
    return [("layer.weight", F32, [3, 5], w32.tobytes()), ("layer.half", F16, [4, 2], w16.tobytes()),
            ("layer.bf", BF16, [7], bf.tobytes()), ("q.int8", I8, [6, 4], q8.tobytes()),
            ("q.int4", I4, [15], q4.tobytes()), ("q.int4.scales", F16, [1], scales.tobytes())]


def mapper_answers(mapper_add, translate, query):
    for alias, hf, aif in RULES:
        mapper_add(alias, hf, aif)
    available = HF_PROBES[:5]
    return {"hf_to_aif": {n: translate(1, n) for n in HF_PROBES}, "aif_to_hf": {n: translate(0, n) for n in AIF_PROBES},
            "missing": query(0, AIF_PROBES, available), "unmapped": query(1, [], HF_PROBES),
            "required": query(2, AIF_PROBES, [])}


def main(out_dir):
    import reflayers as rl
    os.makedirs(out_dir, exist_ok=True)
    m = rl.Mapper()
    answers = mapper_answers(m.add, m.translate, m.query)
    m.close()
    with open(os.path.join(out_dir, "weight_mapper.json"), "w") as f:
        json.dump(answers, f, indent=1, sort_keys=True)
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        rl.st_save(os.path.join(out_dir, "reference_written.safetensors"), format_cases(), METADATA)
    else:
        print("no GPU: reference_written.safetensors not regenerated")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))

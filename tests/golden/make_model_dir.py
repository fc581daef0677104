"""Writes tests/golden/model_tiny/: a model directory produced by the reference's own models/init_model.py
(config.txt + layers/0/combined_layer.weight), for the loader tests.

    python tests/golden/make_model_dir.py <path of the reference checkout>     (or set REFERENCE_ROOT)

One layer, model_dim 64, 1 query / 1 kv head of 32, 8 routed experts of dim 32, top-2, bf16, no vocabulary (so no
embedding or head files), seed 7: about 110 KB.
"""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
CONFIG = {
    "embed_dtype": "bf16", "attn_dtype": "bf16", "router_dtype": "bf16", "expert_dtype": "bf16", "head_dtype": "bf16",
    "vocab_size": 0, "model_dim": 64, "head_dim": 32, "n_layers": 1, "n_heads": 1, "n_kv_heads": 1,
    "qk_norm_type": "none", "qk_norm_weight_type": "none", "num_shared_experts": 0, "num_routed_experts": 8,
    "top_k_routed_experts": 2, "expert_dim": 32, "expert_mlp_type": "swiglu", "rope_theta": 10000,
    "rms_norm_epsilon": 1e-5, "rand_seed": 7,
}


def main():
    if len(sys.argv) < 2 and not os.environ.get("REFERENCE_ROOT"):
        sys.exit("usage: make_model_dir.py <path of the reference checkout>   (or set REFERENCE_ROOT)")
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ["REFERENCE_ROOT"]
    sys.path.insert(0, os.path.join(ref_root, "models"))
    import init_model  # the reference's writer

    out = os.path.join(HERE, "model_tiny")
    with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as fh:
        json.dump(CONFIG, fh)
    init_model.main(fh.name, out)
    os.unlink(fh.name)
    for sub in ("embed", "head"):  # empty when there is no vocabulary
        p = os.path.join(out, sub)
        if os.path.isdir(p) and not os.listdir(p):
            os.rmdir(p)


if __name__ == "__main__":
    main()

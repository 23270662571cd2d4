"""Produce tests/golden/reference_logits.npz from the reference's own CPU model.

Usage:  python tests/golden/make_golden.py /path/to/cuda-inference-serving-runtime

It imports the reference's `runtime` package (NumPy only) from the given checkout,
feeds the tiny random models of tests/tiny_models.py through its `Model.step` one
token at a time (runtime/model.py:86-120: that is the only way it runs a prompt),
and stores the float32 logits of every position.  The reference takes head_dim as
hidden_size // num_attention_heads and has no tied-head switch in `Model`; a tied
model is given the embedding table under both names, as runtime/checkpoint.py:38-39
does.  Nothing of the reference is copied here; the file only calls it.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

CASES = {"tiny_a": ("TINY_A", 11, 40, 101), "tiny_b": ("TINY_B", 12, 48, 102), "tiny_c": ("TINY_C", 13, 24, 103)}


def main(reference_root: str) -> None:
    import tiny_models

    sys.path.insert(0, reference_root)
    from runtime.backend import Backend
    from runtime.model import Config, Model

    out = {}
    for case, (cfg_name, weight_seed, n_tokens, token_seed) in CASES.items():
        cfg = getattr(tiny_models, cfg_name)
        weights = tiny_models.make_weights(cfg, weight_seed)
        if cfg.get("tie_word_embeddings"):
            weights["lm_head.weight"] = weights["model.embed_tokens.weight"]
        fields = ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "rms_norm_eps", "rope_theta", "max_position_embeddings"]
        config = Config(**{k: cfg[k] for k in fields})
        assert config.dim == cfg["head_dim"]
        model = Model(Backend(), config, weights, pages=64, page_size=4)
        model.create("g")
        tokens = tiny_models.random_tokens(cfg, n_tokens, token_seed)
        logits = np.concatenate([model.step([t], ["g"]) for t in tokens]).astype(np.float32)
        out[case + "_tokens"] = np.asarray(tokens, dtype=np.int32)
        out[case + "_logits"] = logits
    np.savez_compressed(HERE / "reference_logits.npz", **out)
    print("wrote", HERE / "reference_logits.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])

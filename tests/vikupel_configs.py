"""Small Vikupel configurations for the tests, and the folder writer they share.

A: sizes that share no factor with the kernels' tiles; key and value heads of different sizes; a
state size that is no multiple of 32; a partial rotation without frequency scaling and values
paired (2m, 2m + 1); a layer without feed-forward; a looped range that holds the recurrent layer
and an attention layer, run three times.
B: everything a multiple of 8, so that 16-bit runs take the tensor-core products; no loop; two
recurrent layers of different shapes; full rotation with scaled frequencies; one KV head under four
query heads, and as many KV heads as query heads.
C: the smallest of everything: a window of one key, a convolution of one tap (no inputs kept), one
head, no token input, a loop that runs once.
"""
import os

VIKUPEL_A = {
    "architecture": "Vikupel", "vocab": 211, "width": 60, "norm": {"eps": 1e-5}, "residual_mult": 0.55,
    "token_side": {"dim": 6}, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 14, "scale": 0.3, "mask": {"size": 19}},
         "mlp": {"kind": "dense", "ff": 100}},
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 6, "state": 20, "groups": 2, "norm_groups": 3, "conv": 3},
         "mlp": {"kind": "dense", "ff": 36}},
        {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.45,
                                          "rot": {"base": 100.0, "dims": 8, "value_layout": "interleaved"}},
         "mlp": {"kind": "dense", "ff": 52}},
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 8, "scale": 0.6,
                                          "rot": {"base": 50.0, "dims": 6,
                                                  "scaling": {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 24}}},
         "mlp": None},
    ],
}
VIKUPEL_B = {
    "architecture": "Vikupel", "vocab": 256, "width": 128, "norm": {"eps": 3e-6}, "residual_mult": 1.3,
    "token_side": {"dim": 8},
    "layers": [
        {"type": "mamba2", "mixer": {"heads": 8, "vdim": 16, "state": 64, "groups": 1, "norm_groups": 1, "conv": 4},
         "mlp": {"kind": "dense", "ff": 256}},
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.18,
                                          "rot": {"base": 10000.0, "dims": 32,
                                                  "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}}},
         "mlp": {"kind": "dense", "ff": 128}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 33}},
         "mlp": {"kind": "dense", "ff": 64}},
        {"type": "mamba2", "mixer": {"heads": 2, "vdim": 64, "state": 16, "groups": 2, "norm_groups": 4, "conv": 2},
         "mlp": None},
    ],
}
VIKUPEL_C = {
    "architecture": "Vikupel", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "loop": {"start": 0, "stop": 3, "times": 1},
    "layers": [
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 1}},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "mamba2", "mixer": {"heads": 1, "vdim": 8, "state": 8, "groups": 1, "norm_groups": 1, "conv": 1}, "mlp": None},
        {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 2, "scale": 0.5,
                                          "rot": {"base": 10.0, "dims": 2}},
         "mlp": {"kind": "dense", "ff": 24}},
    ],
}
VIKUPEL = {"A": (VIKUPEL_A, 3), "B": (VIKUPEL_B, 4), "C": (VIKUPEL_C, 5)}


def write_model(cfg, folder, seed, std=0.12):
    """config.json + model.safetensors (bfloat16 matrices, short tensor names) from the engine's
    random-weights mode; the plain implementation reads the folder with its own reader."""
    from ferrum_b200.weights import write_random_model
    write_random_model(cfg, folder, seed, dtype="bfloat16", std=std)
    assert os.path.exists(os.path.join(folder, "model.safetensors"))
    return folder

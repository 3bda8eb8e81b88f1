"""Small Ruperax configurations for the tests, and the folder writer they share.

A: sizes that share no factor with the kernels' tiles (nothing a multiple of 8 where it can be
avoided), three heads then two then one, a reader layer with fewer heads and a narrower window than
its source, a layer without feed-forward, four norm groups, a window wider than every test sequence.
B: everything a multiple of 8, so that 16-bit runs take the tensor-core products; one norm group,
two source layers with different row sizes (two cache groups), readers of both, a reader with a
wider window than its source.
"""
import os

RUPERAX_A = {
    "architecture": "Ruperax", "vocab": 211, "width": 60, "max_positions": 192,
    "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5, "groups": 4},
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 14, "kv_rank": 22, "q_rank": 18, "scale": 0.31,
                   "mask": {"size": 19}, "rot": {"base": 100.0, "dims": 6}},
         "mlp": {"kind": "dense", "ff": 100}},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 12, "rot_dim": 6, "vdim": 9, "kv_rank": 22, "q_rank": 11, "scale": 0.2, "kv_from": 0,
                   "mask": {"size": 7}, "rot": {"base": 100.0, "dims": 6}},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 1, "dim": 4, "rot_dim": 4, "vdim": 40, "kv_rank": 37, "q_rank": 8, "scale": 0.5,
                   "mask": {"size": 500}, "rot": {"base": 7.0, "dims": 4}},
         "mlp": {"kind": "dense", "ff": 36}},
    ],
}
RUPERAX_B = {
    "architecture": "Ruperax", "vocab": 256, "width": 128, "max_positions": 256,
    "embedding": {"scale": 0.8}, "norm": {"eps": 3e-6, "groups": 1},
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 4, "dim": 32, "rot_dim": 32, "vdim": 64, "kv_rank": 64, "q_rank": 64, "scale": 0.125,
                   "mask": {"size": 48}, "rot": {"base": 10000.0, "dims": 32}},
         "mlp": {"kind": "dense", "ff": 256}},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 64, "rot_dim": 16, "vdim": 32, "kv_rank": 128, "q_rank": 32, "scale": 0.11,
                   "mask": {"size": 33}, "rot": {"base": 500.0, "dims": 16}},
         "mlp": {"kind": "dense", "ff": 128}},
        {"type": "latent_attention",
         "mixer": {"heads": 8, "dim": 16, "rot_dim": 16, "vdim": 16, "kv_rank": 128, "q_rank": 48, "scale": 0.18, "kv_from": 1,
                   "mask": {"size": 40}, "rot": {"base": 500.0, "dims": 16}},
         "mlp": {"kind": "dense", "ff": 64}},
        {"type": "latent_attention",
         "mixer": {"heads": 4, "dim": 32, "rot_dim": 32, "vdim": 24, "kv_rank": 64, "q_rank": 64, "scale": 0.125, "kv_from": 0,
                   "mask": {"size": 16}, "rot": {"base": 10000.0, "dims": 32}},
         "mlp": None},
    ],
}
RUPERAX = {"A": (RUPERAX_A, 3), "B": (RUPERAX_B, 4)}


def write_model(cfg, folder, seed, std=0.12):
    """config.json + model.safetensors (bfloat16 matrices, short tensor names) from the engine's
    random-weights mode; the plain implementation reads the folder with its own reader."""
    from ferrum_b200.weights import write_random_model
    write_random_model(cfg, folder, seed, dtype="bfloat16", std=std)
    assert os.path.exists(os.path.join(folder, "model.safetensors"))
    return folder

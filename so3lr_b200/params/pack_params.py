"""Pack the pretrained SO3LR parameter tree into one flat float32 blob.

Input : so3lr/params/params.pkl of the reference package (a pickled dict of numpy float32 arrays,
        loaded by so3lr/potential.py:17-29 through mlff's `create_from_workdir(from_file=True)`).
Output: so3lr_v1.npz with a single array `blob` (float32) in the fixed order of `LAYOUT` below and
        `sha256` of the source file.  The CUDA library and the CPU oracle both consume this blob, so the
        weights are used bit-exactly as stored in the reference.

Usage: python pack_params.py /path/to/so3lr/params/params.pkl [out.npz]
"""
import hashlib
import pickle
import sys

import numpy as np

NUM_LAYERS = 3


def layout():
    """(key-path, shape) in blob order. Must stay in sync with csrc/params.h."""
    L = []
    L.append(("feature_embeddings_0/Embed_0/embedding", (119, 128)))
    for e in (1, 2):
        p = f"feature_embeddings_{e}/ChargeSpinEmbedSparse_0/"
        L += [(p + "Embed_0/embedding", (119, 128)), (p + "Embed_1/embedding", (2, 128)),
              (p + "Embed_2/embedding", (2, 128)), (p + "Residual_0/layers_0/kernel", (128, 128)),
              (p + "Residual_0/layers_1/kernel", (128, 128))]
    for l in range(NUM_LAYERS):
        a = f"layers_{l}/attention_block/"
        for w in ("Wq1", "Wk1", "Wv1", "Wq2", "Wk2"):
            L.append((a + w, (4, 32, 32)))
        for f in (1, 2):
            L += [(a + f"radial_filter{f}_layer_1/kernel", (32, 128)), (a + f"radial_filter{f}_layer_1/bias", (128,)),
                  (a + f"radial_filter{f}_layer_2/kernel", (128, 128)), (a + f"radial_filter{f}_layer_2/bias", (128,))]
        for f in (1, 2):
            L += [(a + f"spherical_filter{f}_layer_1/kernel", (4, 32)), (a + f"spherical_filter{f}_layer_1/bias", (32,)),
                  (a + f"spherical_filter{f}_layer_2/kernel", (32, 128)), (a + f"spherical_filter{f}_layer_2/bias", (128,))]
        b = f"layers_{l}/"
        L += [(b + "exchange_block/mlp_layer_2/kernel", (132, 132)), (b + "exchange_block/mlp_layer_2/bias", (132,)),
              (b + "layer_normalization_1/scale", (128,)), (b + "layer_normalization_1/bias", (128,)),
              (b + "layer_normalization_2/scale", (128,)), (b + "layer_normalization_2/bias", (128,)),
              (b + "res_mlp_1_layer_1/kernel", (128, 128)), (b + "res_mlp_1_layer_1/bias", (128,)),
              (b + "res_mlp_1_layer_2/kernel", (128, 128)), (b + "res_mlp_1_layer_2/bias", (128,))]
    o = "observables_0/"
    L += [(o + "energy_dense_regression/kernel", (128, 128)), (o + "energy_dense_regression/bias", (128,)),
          (o + "energy_dense_final/kernel", (128, 1)), (o + "energy_dense_final/bias", (1,)),
          (o + "atomic_scales", (119,)), (o + "energy_offset", (119,))]
    for k in ("a1", "a2", "a3", "a4", "c1", "c2", "c3", "c4", "p", "d"):
        L.append((o + "zbl_repulsion/" + k, (1,)))
    q = o + "electrostatic_energy/partial_charges/"
    L += [(q + "Embed_0/embedding", (100, 1)), (q + "charge_dense_regression_vec/kernel", (128, 128)),
          (q + "charge_dense_regression_vec/bias", (128,)), (q + "charge_dense_final_vec/kernel", (128, 1)),
          (q + "charge_dense_final_vec/bias", (1,))]
    h = "observables_2/"
    L += [(h + "Embed_0/embedding", (100, 1)), (h + "Embed_1/embedding", (100, 64)),
          (h + "hirshfeld_ratios_dense_regression/kernel", (128, 64)), (h + "hirshfeld_ratios_dense_regression/bias", (64,)),
          (h + "hirshfeld_ratios_dense_final/kernel", (64, 64)), (h + "hirshfeld_ratios_dense_final/bias", (64,))]
    return L


def offsets():
    off, out = 0, {}
    for k, shp in layout():
        out[k] = (off, shp)
        off += int(np.prod(shp))
    return out, off


def unpack(blob):
    """blob -> {key-path: ndarray view}"""
    offs, total = offsets()
    assert blob.size == total, (blob.size, total)
    return {k: blob[o:o + int(np.prod(s))].reshape(s) for k, (o, s) in offs.items()}


def pack(tree):
    parts = []
    for k, shp in layout():
        node = tree
        for part in k.split("/"):
            node = node[part]
        a = np.asarray(node, dtype=np.float32)
        assert a.shape == tuple(shp), (k, a.shape, shp)
        parts.append(a.ravel())
    return np.concatenate(parts)


if __name__ == "__main__":
    src = sys.argv[1]
    dst = sys.argv[2] if len(sys.argv) > 2 else "so3lr_v1.npz"
    raw = open(src, "rb").read()
    tree = pickle.loads(raw)["params"]
    blob = pack(tree)
    n_leaves = len(layout())
    np.savez_compressed(dst, blob=blob, sha256=hashlib.sha256(raw).hexdigest(), n_leaves=n_leaves)
    print(f"packed {n_leaves} leaves, {blob.size} float32 -> {dst}")

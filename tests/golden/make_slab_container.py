"""Writes a small weight container in the engine's on-disk layout for the
slab-loader tests: shards with each expert's slab {gate_up [2I,H] | down
[H,I]} contiguous at some offset among other bytes, and the manifest
apus.index.json (format_version 2) with a tensor_map and the expert_slabs
records {layer, expert, shard, offset, nbytes} (the reference's
tools/convert.py:880-940 writes the same members).  Used at test time into a
temporary directory; nothing large is committed.

    python tests/golden/make_slab_container.py OUT_DIR   # a demo container
"""
import json
import os
import sys

import numpy as np


def write_container(out_dir, layers, H, I, n_shards=2, seed=0, version=2,
                    drop=None, truncate=None):
    """layers: {layer_index: (exp_gu [E,2I,H] uint16, exp_d [E,H,I] uint16)}.
    Experts are spread round-robin over n_shards shard files, each slab
    preceded by a run of unrelated bytes.  drop: (layer, expert) left out of
    the manifest; truncate: (layer, expert) recorded one byte short."""
    rng = np.random.default_rng(seed)
    os.makedirs(out_dir, exist_ok=True)
    names = [f"apus-qwen-{i + 1:05d}.safetensors" for i in range(n_shards)]
    files = [open(os.path.join(out_dir, n), "wb") for n in names]
    for f in files:                       # a safetensors-like preamble
        hdr = json.dumps({"__metadata__": {"format": "pt", "note": "fixture {[\"}]"}}).encode()
        f.write(len(hdr).to_bytes(8, "little") + hdr)
    slabs, tensor_map = [], {}
    k = 0
    for layer, (gu, d) in sorted(layers.items()):
        E = gu.shape[0]
        for e in rng.permutation(E):
            s = k % n_shards
            k += 1
            f = files[s]
            f.write(rng.integers(0, 256, int(rng.integers(1, 5000)), dtype=np.uint8).tobytes())
            off = f.tell()
            f.write(np.ascontiguousarray(gu[e]).tobytes())
            f.write(np.ascontiguousarray(d[e]).tobytes())
            nbytes = f.tell() - off
            base = f"model.language_model.layers.{layer}.mlp.experts.{int(e)}."
            tensor_map[base + "gate_up_proj.weight"] = {
                "shard": names[s], "offset": off, "nbytes": gu[e].nbytes,
                "dtype": "BF16", "shape": [2 * I, H]}
            tensor_map[base + "down_proj.weight"] = {
                "shard": names[s], "offset": off + gu[e].nbytes, "nbytes": d[e].nbytes,
                "dtype": "BF16", "shape": [H, I]}
            if drop == (layer, int(e)):
                continue
            slabs.append({"layer": int(layer), "expert": int(e), "shard": names[s],
                          "offset": off,
                          "nbytes": nbytes - (1 if truncate == (layer, int(e)) else 0)})
    # a record of a layer this model does not have (the speculative block's
    # numbering, c/cache.h:25-31): the loader must skip it
    slabs.append({"layer": 10_000, "expert": 0, "shard": names[0], "offset": 8, "nbytes": 16})
    for f in files:
        f.close()
    manifest = {"format_version": version, "config_hash": "fixture \"quoted\" \\ {",
                "offset_base": "file", "header_reserve": 0,
                "shard_groups": {"main": names, "mtp": []},
                "ntensors": len(tensor_map), "tensor_map": tensor_map,
                "expert_slabs": slabs, "stripped_tensors": 0}
    with open(os.path.join(out_dir, "apus.index.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    return manifest


if __name__ == "__main__":
    H, I, E = 128, 32, 16
    r = np.random.default_rng(1)
    write_container(sys.argv[1], {0: (r.integers(0, 1 << 16, (E, 2 * I, H), dtype=np.uint16),
                                      r.integers(0, 1 << 16, (E, H, I), dtype=np.uint16))},
                    H, I)
    print("wrote", sys.argv[1])

#!/usr/bin/env python3
"""Regenerates the committed golden fixtures under tests/golden/.

Run where a checkout of the reference exists (environment variable REF names
it); the fixtures it writes are what travels.  Three families:

  m4a/      the reference's own per-op MoE goldens: its generator
            tests/m4a/gen_golden.py is imported unmodified and run with its
            fixed seed into a scratch directory; the MoE files and the MoE
            keys of its manifest are kept.
  block_*   MoE-block outputs of the reference's own compiled C code
            (oracle/_ref/libapus_ref.so: apus_layer_moe / apus_layer_moe_batch)
            on seeded synthetic weights: inputs, selected ids, routing
            weights, routed/shared/out stages, plus a checksum of the weights
            so a drifting generator is caught.
  npblock   the reference's independent numpy oracle (tools/oracle.py
            moe_forward, f32 mode) on the mini configuration.
"""
import hashlib
import importlib.util
import os
import shutil
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("REF", "/root/reference")
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def weights_digest(W):
    h = hashlib.sha256()
    for k in sorted(W):
        h.update(W[k].tobytes())
    return h.hexdigest()


def gen_m4a():
    gg = load(os.path.join(REF, "tests/m4a/gen_golden.py"), "ref_gen_golden")
    tmp = tempfile.mkdtemp()
    gg.OUT = tmp
    gg.main()
    out = os.path.join(HERE, "m4a")
    os.makedirs(out, exist_ok=True)
    for f in sorted(os.listdir(tmp)):
        if f.startswith("moe_"):
            shutil.copy(os.path.join(tmp, f), os.path.join(out, f))
    keep = ("RTR_", "ACT_", "SILU_", "COMB_")
    with open(os.path.join(tmp, "manifest.txt")) as src, \
            open(os.path.join(out, "manifest.txt"), "w") as dst:
        for line in src:
            if line.startswith(keep):
                dst.write(line)
    shutil.rmtree(tmp)


def gen_blocks():
    import conftest
    from oracle import oracle
    pkg = conftest.load_package()
    pkg.build.build()
    be = pkg.Backend()
    import apus_b200.synth as synth
    oracle.build()
    ref = oracle.Reference()
    cases = [
        ("block_mini_t7", synth.MINI_CFG, 7, 11, 0.08),
        ("block_mini_t1", synth.MINI_CFG, 1, 12, 0.08),
        ("block_qwen_t3", synth.QWEN_CFG, 3, 0, 0.02),
    ]
    for name, cfg, T, seed, sigma in cases:
        W = synth.host_weights(be, cfg, seed=seed, sigma=sigma)
        x = synth.host_x(be, T, cfg["hidden"], seed=seed)
        r = ref.moe_block(cfg, W, x, batched=T > 1)
        # the per-token body must agree with the batched body (tests/m9c)
        r1 = ref.moe_block(cfg, W, x, batched=False)
        for k in r:
            assert np.array_equal(r[k], r1[k]), (name, k)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            cfg=np.array([cfg[k] for k in ("hidden", "experts", "moe_inter",
                                            "shared_inter", "top_k")]),
            seed=seed, sigma=sigma, x=x, digest=weights_digest(W), **r)
        print(name, "idx[0] =", r["idx"][0].tolist())

    # numpy oracle on the mini configuration
    orc = load(os.path.join(REF, "tools/oracle.py"), "ref_np_oracle")
    cfg = synth.MINI_CFG
    W = synth.host_weights(be, cfg, seed=11, sigma=0.08)
    x = synth.host_x(be, 7, cfg["hidden"], seed=11)
    ncfg = dict(orc.MINI_CFG)
    ncfg.update(hidden_size=cfg["hidden"], num_experts=cfg["experts"],
                moe_intermediate_size=cfg["moe_inter"],
                shared_expert_intermediate_size=cfg["shared_inter"],
                num_experts_per_tok=cfg["top_k"])
    Wf = {k: synth.bf16_to_f32(v).astype(np.float64) for k, v in W.items()}
    outs, idxs = [], []
    for t in range(x.shape[0]):
        xv = synth.bf16_to_f32(x[t]).astype(np.float64)
        r = orc.moe_forward(xv, Wf, orc.f32, orc.rnd16, ncfg)
        outs.append(r["out"])
        idxs.append(r["idx"])
    np.savez_compressed(os.path.join(HERE, "npblock_mini_t7.npz"),
                        out=np.array(outs), idx=np.array(idxs))
    print("npblock idx[0] =", idxs[0].tolist())


if __name__ == "__main__":
    gen_m4a()
    gen_blocks()

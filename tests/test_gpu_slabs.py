"""Routed-expert weights straight from the engine's weight container
(apus.index.json + shards, c/cache.h:13-23) into HBM, for a rank's expert
range, against the engine's eager load, which concatenates the same slab bytes
into host arrays first (c/model.h:505-537): the block computed from either
must be the same bit for bit."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_slab_container import write_container   # noqa: E402

pytestmark = pytest.mark.gpu

CFG = dict(hidden=512, experts=16, moe_inter=128, shared_inter=128, top_k=4)


def _layers(be, synth, n=2):
    Ws = [synth.host_weights(be, CFG, seed=70, layer=l, sigma=0.05) for l in range(n)]
    return Ws, {l: (W["exp_gu"], W["exp_d"]) for l, W in enumerate(Ws)}


def test_layer_from_slabs_equals_layer_from_host_arrays(gpu, be, synth, tmp_path):
    import torch
    Ws, layers = _layers(be, synth)
    write_container(tmp_path, layers, CFG["hidden"], CFG["moe_inter"], n_shards=3)
    T = 40
    x = synth.host_x(be, T, CFG["hidden"], seed=70)
    d_x = torch.from_numpy(x.view(np.int16)).cuda()
    for l in (0, 1):
        ref_layer = gpu.layer_create(CFG, Ws[l])
        up0 = gpu.bytes_uploaded()
        lay = gpu.layer_create(CFG, None)
        for name in ("rtr_w", "sh_g", "sh_u", "sh_d", "sh_gate"):
            gpu.layer_upload(lay, name, Ws[l][name])
        up1 = gpu.bytes_uploaded()
        gpu.layer_load_slabs(lay, tmp_path, l)
        assert gpu.bytes_uploaded() - up1 == Ws[l]["exp_gu"].nbytes + Ws[l]["exp_d"].nbytes
        outs = []
        for h in (ref_layer, lay):
            o = torch.empty_like(d_x)
            gpu.moe_block_dev(h, d_x.data_ptr(), o.data_ptr(), T)
            torch.cuda.synchronize()
            outs.append(o.cpu().numpy())
        assert np.array_equal(outs[0], outs[1])
        assert up1 > up0


def test_a_rank_loads_only_its_own_experts(gpu, be, synth, tmp_path):
    """Expert range [4, 12): the resident tensors equal that slice of the
    eager arrays (checked through apus_cuda_experts_dev on rows of those
    experts)."""
    import torch
    Ws, layers = _layers(be, synth, 1)
    write_container(tmp_path, layers, CFG["hidden"], CFG["moe_inter"])
    W = Ws[0]
    a = gpu.layer_create(CFG, W, 4, 12)
    b = gpu.layer_create(CFG, None, 4, 12)
    gpu.layer_load_slabs(b, tmp_path, 0)
    R = 64
    rng = np.random.default_rng(2)
    e = torch.from_numpy(rng.integers(4, 12, R).astype(np.int32)).cuda()
    x = torch.from_numpy(synth.host_x(be, R, CFG["hidden"], seed=3).view(np.int16)).cuda()
    ys = []
    for h in (a, b):
        y = torch.empty_like(x)
        gpu.experts_dev(h, x.data_ptr(), e.data_ptr(), R, y.data_ptr())
        torch.cuda.synchronize()
        ys.append(y.cpu().numpy())
    assert np.array_equal(ys[0], ys[1])


@pytest.mark.parametrize("kind", ["no_manifest", "version", "missing_record",
                                  "wrong_size", "missing_shard", "garbage"])
def test_bad_containers_are_refused(gpu, be, synth, tmp_path, kind):
    Ws, layers = _layers(be, synth, 1)
    kw = {}
    if kind == "version":
        kw["version"] = 1
    elif kind == "missing_record":
        kw["drop"] = (0, 5)
    elif kind == "wrong_size":
        kw["truncate"] = (0, 7)
    if kind != "no_manifest":
        write_container(tmp_path, layers, CFG["hidden"], CFG["moe_inter"], **kw)
    if kind == "missing_shard":
        os.remove(os.path.join(tmp_path, "apus-qwen-00002.safetensors"))
    if kind == "garbage":
        with open(os.path.join(tmp_path, "apus.index.json"), "w") as f:
            f.write('{"format_version": 2, "expert_slabs": [ {"layer": 0, ')
    lay = gpu.layer_create(CFG, None)
    with pytest.raises(Exception) as ei:
        gpu.layer_load_slabs(lay, tmp_path, 0)
    msg = str(ei.value)
    want = {"no_manifest": "cannot open", "version": "format_version",
            "missing_record": "no slab record", "wrong_size": "expected",
            "missing_shard": "cannot open shard", "garbage": "malformed"}[kind]
    assert want in msg, msg
    # the backend stays usable
    gpu.layer_destroy(lay)


def test_tiered_layer_registered_from_the_container(gpu, orc, be, synth, tmp_path):
    """The engine's tiered mode has no expert arrays on the host; the layer is
    registered once from the container and the host-pointer block call then
    serves it under the same key with exp_gu / exp_d NULL: same result, bit for
    bit, as the eager call with the arrays."""
    Ws, layers = _layers(be, synth, 1)
    W = Ws[0]
    write_container(tmp_path, layers, CFG["hidden"], CFG["moe_inter"])
    x = synth.host_x(be, 33, CFG["hidden"], seed=9)
    eager = gpu.moe_block(CFG, W, x)
    # a second set of host pointers for the non-expert tensors = a second key
    Wt = {k: (v.copy() if k not in ("exp_gu", "exp_d") else None) for k, v in W.items()}
    with pytest.raises(Exception) as ei:
        gpu.moe_block(CFG, Wt, x)
    assert "register_layer_slabs" in str(ei.value)
    gpu.register_layer_slabs(CFG, Wt, tmp_path, 0)
    gpu.register_layer_slabs(CFG, Wt, tmp_path, 0)        # idempotent
    tiered = gpu.moe_block(CFG, Wt, x)
    for k in ("idx", "w", "routed", "shared", "out"):
        assert np.array_equal(eager[k], tiered[k]), k
    exp = orc.moe_block(CFG, W, x)
    assert np.array_equal(tiered["idx"], exp["idx"])

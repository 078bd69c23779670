"""The engine-side glue (include/apus_cuda_glue.h) compiled into the reference
engine's own translation unit (oracle/glue_harness.c -> oracle/_ref/glue_test,
linked against libapus_cuda.so as the engine's -cuda binary would be).  The
programs are built where the reference checkout exists and travel with the
tree; the tests run them."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GLUE = os.path.join(ROOT, "oracle", "_ref", "glue_test")
GLUE_CPU = os.path.join(ROOT, "oracle", "_ref", "glue_test_cpu")


def run(exe, *args, env=None):
    if not os.path.exists(exe):
        pytest.skip(f"{os.path.basename(exe)} not built (needs the reference checkout)")
    e = dict(os.environ)
    e.update(env or {})
    p = subprocess.run([exe, *map(str, args)], capture_output=True, text=True,
                       env=e, timeout=600)
    line = [l for l in p.stdout.splitlines() if l.startswith("{")]
    return p.returncode, (json.loads(line[-1]) if line else None), p.stderr


def test_glue_header_is_c11(tmp_path):
    src = tmp_path / "t.c"
    src.write_text(
        '#include <stddef.h>\n#include <stdint.h>\n'
        'typedef struct { size_t hidden, experts, moe_inter, shared_inter, top_k; } ApusLayerCfg;\n'
        'typedef struct { const uint16_t *rtr_w, *exp_gu, *exp_d, *sh_g, *sh_u, *sh_d, *sh_gate; } ApusLayerW;\n'
        'typedef struct { int32_t *rtr_idx; uint16_t *rtr_w, *moe_routed, *moe_shared, *moe_out; } ApusLayerTrace;\n'
        '#define APUS_CUDA_GLUE_WEAK_STUBS\n#include "apus_cuda_glue.h"\n'
        'int main(void){ApusLayerCfg c = {0,0,0,0,0}; ApusLayerW w = {0,0,0,0,0,0,0};\n'
        'return apus_layer_moe_cuda(&c, &w, 0, 0, 1, 0, 0) == 1 ? 0 : 1;}\n')
    exe = tmp_path / "t"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror",
                    "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)],
                   check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_cpu_only_binary_links_and_says_not_compiled_in():
    rc, j, _ = run(GLUE_CPU, "stubs")
    assert rc == 0
    assert j["enable_rc"] == -1 and "not compiled in" in j["err"]
    assert j["shim_rc"] == 1 and j["topn_rc"] == 1 and j["enabled"] == 0


def test_cuda_binary_without_a_device_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    rc, j, _ = run(GLUE, "slots")
    assert rc != 0 and "error" in j


@pytest.mark.gpu
@pytest.mark.parametrize("shape,T,t0", [
    ((128, 16, 32, 32, 4), 1, 5), ((128, 16, 32, 32, 4), 7, 0),
    ((512, 64, 128, 128, 8), 3, 2), ((512, 64, 128, 128, 8), 150, 9)])
def test_shim_inside_the_engine_matches_its_cpu_block(shape, T, t0):
    """apus_layer_moe_cuda with real ApusLayerCfg / W / Trace objects against
    the engine's own apus_layer_moe_batch: ids exact, outputs to BF16
    tolerance, trace rows written at offset t0 and nowhere before it."""
    rc, j, err = run(GLUE, "block", *shape, T, t0)
    assert rc == 0, err
    assert j["rc"] == 0 and j["idx_exact"] == 1
    assert j["w_codes_differing"] <= max(1, T * shape[4] // 100)
    assert j["max_abs"] <= 2e-2 and j["rel_l2"] <= 1e-2
    assert j["max_abs_routed"] <= 2e-2 and j["max_abs_shared"] <= 2e-2
    assert j["rows_before_t0_untouched"] == 1 and j["trace_out_equals_out"] == 1
    assert j["launches"] > 0


@pytest.mark.gpu
def test_enable_fills_the_engines_own_table_and_knobs_leave_slots_null():
    rc, j, err = run(GLUE, "slots")
    assert rc == 0, err
    assert j == {"gemv": 1, "gemm": 1, "matvec": 1, "moe": 1, "enabled": 1}
    for knob, slot in (("APUS_CUDA_NO_GEMV", "gemv"), ("APUS_CUDA_NO_GEMM", "gemm"),
                       ("APUS_CUDA_NO_MATVEC", "matvec"), ("APUS_CUDA_NO_MOE", "moe")):
        rc, j, err = run(GLUE, "slots", env={knob: "1"})
        assert rc == 0, err
        assert j[slot] == 0
        assert sum(j[s] for s in ("gemv", "gemm", "matvec", "moe")) == 3


@pytest.mark.gpu
def test_budget_exhausted_hook_declines_and_the_engine_falls_back():
    """The reference's fail-soft idiom: the hook returns nonzero, the engine's
    hot wrapper runs its CPU kernel, the result is still the anchor's."""
    rc, j, err = run(GLUE, "budget", 256, 512)
    assert rc == 0, err
    assert j["hook_took_it"] == 1 and j["bitwise_scalar"] == 1
    rc, j, err = run(GLUE, "budget", 1024, 1024, env={"APUS_CUDA_DENSE_MB": "1"})
    assert rc == 0, err
    assert j["hook_took_it"] == 0 and j["bitwise_scalar"] == 1
    assert j["bytes_resident"] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("E,K,n", [(16, 128, 4), (256, 2048, 8), (256, 2048, 12)])
def test_predictor_router_truncation_through_the_glue(E, K, n):
    """c/pilot.h:280-284: the first n expert ids in selection order."""
    rc, j, err = run(GLUE, "topn", E, K, n)
    assert rc == 0, err
    assert j["rc"] == 0 and j["equal"] == 1 and j["launches"] > 0

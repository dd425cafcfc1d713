"""install()/uninstall() rebind the reference's module-level operator names (checked against a stand-in package tree;
the reference itself is not needed)."""
import importlib
import sys
import types

import pytest


@pytest.fixture
def fake_reference(monkeypatch):
    names = {
        "easyvolcap": [],
        "easyvolcap.utils": [],
        "easyvolcap.utils.custom_indexer": ["sparse_topk_indexer_func", "sparse_topk_indexer_inference_func"],
        "easyvolcap.utils.custom_flash_attn": [],
        "easyvolcap.utils.custom_flash_attn.sparse_index_flash_attn": [
            "sparse_index_flash_attn_func", "sparse_index_flash_attn_bhtd_func", "dense_index_flash_attn_func",
            "sparse_index_flash_attn_inference_func", "sparse_index_flash_attn_inference_bhtd_func",
            "sparse_index_flash_attn_value_gate_bhtd_func"],
        "easyvolcap.official_vggt": [],
        "easyvolcap.official_vggt.layers": [],
        "easyvolcap.official_vggt.layers.indexer": ["sparse_topk_indexer_func", "sparse_topk_indexer_inference_func"],
        "easyvolcap.official_vggt.layers.dsa_attention": [
            "sparse_index_flash_attn_func", "sparse_index_flash_attn_bhtd_func", "dense_index_flash_attn_func",
            "sparse_index_flash_attn_inference_func", "sparse_index_flash_attn_inference_bhtd_func",
            "sparse_index_flash_attn_value_gate_bhtd_func"],
    }
    for name, attrs in names.items():
        mod = types.ModuleType(name)
        mod.__path__ = []
        for a in attrs:
            setattr(mod, a, None if a == "sparse_topk_indexer_inference_func" else f"reference:{a}")
        monkeypatch.setitem(sys.modules, name, mod)
    return names


def test_install_rebinds_every_operator_and_uninstall_restores(fake_reference):
    import geoweave_b200
    from geoweave_b200 import build as gw_build

    gw_build.build()
    patched = geoweave_b200.install()
    assert len(patched) == 16
    idx_mod = sys.modules["easyvolcap.official_vggt.layers.indexer"]
    dsa_mod = sys.modules["easyvolcap.official_vggt.layers.dsa_attention"]
    ours_idx = importlib.import_module("geoweave_b200.custom_indexer")
    ours_att = importlib.import_module("geoweave_b200.custom_flash_attn")
    assert idx_mod.sparse_topk_indexer_func is ours_idx.sparse_topk_indexer_func
    assert idx_mod.sparse_topk_indexer_inference_func is ours_idx.sparse_topk_indexer_inference_func  # the open slot
    assert dsa_mod.sparse_index_flash_attn_inference_func is ours_att.sparse_index_flash_attn_inference_func
    assert sys.modules["easyvolcap.utils.custom_indexer"].sparse_topk_indexer_func is ours_idx.sparse_topk_indexer_func
    geoweave_b200.uninstall()
    assert idx_mod.sparse_topk_indexer_func == "reference:sparse_topk_indexer_func"
    assert idx_mod.sparse_topk_indexer_inference_func is None
    assert dsa_mod.sparse_index_flash_attn_func == "reference:sparse_index_flash_attn_func"


def test_cpu_tensors_are_refused_not_silently_computed():
    import torch

    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_inference_func
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    q = torch.zeros(1, 4, 4, 64, dtype=torch.bfloat16)
    w = torch.zeros(1, 4, 4, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        sparse_topk_indexer_func(q, q, w, None, 2, None, 0)
    with pytest.raises(ValueError):
        sparse_index_flash_attn_inference_func(q, q, q, torch.zeros(1, 4, 2, dtype=torch.int32))


def test_reference_arm_of_the_benchmark_prints_one_json_line():
    import json
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "small",
                          "--cpu-rows", "64", "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    from baseline import ref_harness

    # the reference's own functions when its sources are staged under baseline/_ref, the oracle's port otherwise
    assert line["cpu_baseline"]["kind"] == ("reference" if ref_harness.available() else "port")
    assert line["e2e"]["h2d_bytes_per_step"] == 0

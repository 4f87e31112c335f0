"""CPU: the benchmark's command line — the reference arm prints the contracted JSON line, and
the host-side helpers behave."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == "GB/s"
    assert d["higher_is_better"] is True and d["steps"] == 2 and d["gpu_launches"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["bytes_per_step"] == 64 << 20 and d["value"] > 0
    # both arms describe the workload with the very same dictionary
    assert d["config"] == bench.headline_config()
    assert d["run"]["timing"]["rounds"] >= 3 and d["run"]["timing"]["steps_per_round"] == 2


def test_reference_arm_does_not_load_the_product_library():
    """The CPU arm times the oracle port; it must not map the product's shared objects."""
    code = ("import sys; sys.argv=['bench.py','--impl','reference','--steps','1','--warmup','3'];"
            "import runpy; runpy.run_path(%r, run_name='__main__');"
            "maps=open('/proc/self/maps').read();"
            "assert 'liblmserve_kv' not in maps and '_packer' not in maps, 'product .so mapped';"
            "assert 'lmserve_b200' not in sys.modules") % str(ROOT / "bench.py")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]


def test_rounds_per_graph_targets_two_milliseconds():
    assert bench.rounds_per_graph(20, 11.0) == 10           # 10 x 20 x 11 us = 2.2 ms
    assert bench.rounds_per_graph(200, 11.0) == 1            # one round is already 2.2 ms
    assert bench.rounds_per_graph(1, 11.0) == 182
    assert bench.rounds_per_graph(1, 0.5) == 512             # capped by the node count
    assert bench.rounds_per_graph(1000, 11.0) == 1           # never less than one round


def test_profile_traffic_follows_the_kernel():
    val, src = bench.profile_traffic("write_rows_direct")
    assert val is None or (val > 1e6 and src.startswith("write_rows_direct"))
    assert bench.profile_traffic("no_such_kernel") == (None, None)


def test_reference_arm_other_ranks_stay_silent():
    import os
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1"], capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_our_arm_refuses_to_run_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1"], capture_output=True,
                         text=True, timeout=120, cwd=ROOT)
    assert out.returncode != 0 and "no CPU path" in (out.stderr + out.stdout)


def test_renumber_blocks_keeps_structure():
    import workloads as W
    w = W.config2()
    new = bench.renumber_blocks(w.slot_mapping, 16, 2048, seed=3)
    assert new.max() < 2048 * 16 and len(np.unique(new)) == len(new)
    assert np.array_equal(new % 16, w.slot_mapping % 16)                # entry inside the block kept
    # tokens that shared a block still share one, and only those
    old_b, new_b = w.slot_mapping // 16, new // 16
    assert len(np.unique(old_b)) == len(np.unique(new_b))
    assert len(set(zip(old_b.tolist(), new_b.tolist()))) == len(np.unique(old_b))


def test_host_pool_blocks_respects_the_cap():
    per_block = 32 * 65536
    assert bench.host_pool_blocks(per_block, 131072, 32.0) <= 16384
    n = bench.host_pool_blocks(per_block, 131072, 1.0)
    assert n * per_block <= 1 << 30 and n >= 1 and (n & (n - 1)) == 0


def test_compact_decode_cases_are_the_same_steps():
    import workloads as W
    w, shape, slots = bench.compact_decode_cases(3)
    originals = [W.config2(seed=1002 + 17 * i).slot_mapping for i in range(3)]
    assert shape.num_blocks == len(np.unique(np.concatenate(originals) // 16))
    for got, want in zip(slots, originals):
        assert np.array_equal(got % 16, want % 16) and len(np.unique(got)) == 256
        assert got.max() < shape.num_blocks * 16
        # tokens that shared a block still share one
        assert len(set(zip((want // 16).tolist(), (got // 16).tolist()))) == len(np.unique(want // 16))

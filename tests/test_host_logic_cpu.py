"""CPU: host-side pieces around the kernels -- the permutation cache, the timing table, and the
reference arm of the benchmark (which must run without the product and on every core)."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_permutation_cache_is_keyed_by_content_not_by_address():
    from dfsattn_b200.engine import PermutationCache
    cache = PermutationCache(max_entries=3)
    cpu = torch.device("cpu")
    a = torch.tensor([2, 0, 1, 3])
    perm_a, inv_a = cache.get(a, 6, 4, cpu)
    assert perm_a.tolist() == [2, 0, 1, 3, 4, 5] and inv_a.tolist() == [1, 2, 0, 3, 4, 5]
    assert cache.get(a, 6, 4, cpu)[0] is perm_a                       # same object: hit
    assert cache.get(a.clone(), 6, 4, cpu)[0] is perm_a               # equal content in a new tensor: hit
    b = torch.tensor([3, 2, 1, 0])                                    # same length, other content: no alias
    assert cache.get(b, 6, 4, cpu)[0].tolist() == [3, 2, 1, 0, 4, 5]
    a[0], a[1] = 0, 2                                                 # modified in place: rebuilt
    assert cache.get(a, 6, 4, cpu)[0].tolist() == [0, 2, 1, 3, 4, 5]
    for i in range(5):                                                # bounded
        cache.get(torch.roll(torch.arange(4), i), 6, 4, cpu)
    assert len(cache._cache) <= 3
    assert cache.get(None, 6, 4, cpu) == (None, None)


def test_timing_table_has_the_reference_columns_and_categories(tmp_path):
    from dfsattn_b200.timing import AttentionTimingRecorder
    rec = AttentionTimingRecorder(enabled=True)
    for phase in ("topk_mask", "topk_routing", "attention_execution", "attention_execution"):
        rec.stop(rec.start("cpu"), phase=phase, step_idx=0, layer_idx=0, device="cpu")
    table = rec.dump_csv(str(tmp_path / "t.csv"), extra_totals={"e2e_gpu": 12.5})
    assert table["top_k_selection"]["calls"] == 1 and table["attention_execution"]["calls"] == 2
    assert "topk_routing" not in table and table["e2e_gpu"]["total_ms"] == 12.5
    lines = (tmp_path / "t.csv").read_text().splitlines()
    assert lines[0] == "phase,total_ms,calls,mean_ms"
    assert [ln.split(",")[0] for ln in lines[1:]] == ["top_k_selection", "attention_execution", "e2e_gpu"]


def test_reference_arm_runs_without_the_product_and_on_all_cores():
    code = ("import runpy, sys, os\n"
            "sys.argv = ['bench.py', '--impl', 'reference', '--workload', 'tiny', '--steps', '1', '--warmup', '0',"
            " '--cpu-blocks', '4', '--gpus', '2']\n"
            "runpy.run_path(os.path.join(%r, 'bench.py'), run_name='__main__')\n"
            "bad = [m for m in sys.modules if m == 'dfsattn_b200' or m.startswith('dfsattn_b200.')]\n"
            "maps = open('/proc/self/maps').read()\n"
            "assert not bad and 'libdfs_b200' not in maps, (bad, 'libdfs_b200' in maps)\n") % ROOT
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
    env.pop("DFSATTN_REFERENCE_PATH", None)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT,
                         timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["gpu_launches"] == 0 and line["n_gpus"] == 2
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))       # not torchrun's single thread
    assert line["config"]["workload"] == "tiny" and line["config"]["heads"] == 2 and "sample" in line["config"]
    # another rank of the same launch prints nothing
    env["RANK"] = "1"
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "tiny",
                          "--steps", "1", "--warmup", "0", "--gpus", "2"], capture_output=True, text=True, env=env,
                         cwd=ROOT, timeout=600)
    assert out.returncode == 0 and out.stdout.strip() == ""

"""Host-side pieces of bench.py that need no GPU: the clock sampler's windows and throttle
reasons, the decode batch of the benchmark, the reference arm on a rank that must stay idle."""
import os
import subprocess
import sys

import numpy as np

import bench
from relay_b200.types import flatten

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_clock_sampler_reads_only_the_rows_of_its_window():
    s = bench.ClockSampler(0)
    s.rows = [(1.0, ["1900", "1965", "300", "Not Active", "Not Active", "Not Active", "Not Active"]),
              (2.0, ["1650", "1965", "990", "Not Active", "Not Active", "Not Active", "Active"]),
              (2.1, ["1700", "1965", "995", "Not Active", "Not Active", "Not Active", "Active"]),
              (2.2, ["1710", "1965", "[N/A]", "Not Active", "Not Active", "Not Active", "Active"]),
              (3.5, ["600", "1965", "100", "Active", "Not Active", "Not Active", "Not Active"]),
              (3.6, ["garbage"])]
    assert s.count(1.5, 2.5) == 3
    d = s.summary(1.5, 2.5)
    assert d == {"sm_mhz": 1700.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    assert s.summary(3.0, 4.0)["reasons"] == ["hw_slowdown"] and s.summary(3.0, 4.0)["samples"] == 1
    assert s.summary(10.0, 11.0) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


def test_decode_batch_is_one_token_per_sequence_over_disjoint_block_tables():
    b = bench.decode_batch(8, 100, 16, 1000, seed=3)
    fb = flatten(b)
    assert fb.n_seqs == 8 and fb.n_tokens == 8 and fb.n_rows == 8
    assert np.all(fb.chunk_len == 1) and np.all(fb.start_pos == 99)
    assert np.all(fb.table_len == 7)  # ceil(100 / 16)
    assert len(set(fb.tables.tolist())) == 8 * 7  # a permutation of the pool: no block twice


def test_bind_to_gpu_cores_is_harmless_without_nvml_devices():
    before = os.sched_getaffinity(0)
    got = bench.bind_to_gpu_cores(0)
    assert got is None or got > 0
    os.sched_setaffinity(0, before)


def test_reference_arm_stays_idle_on_other_ranks():
    env = dict(os.environ, WORLD_SIZE="2", RANK="1", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_step_bytes_count_kv_once_and_weights_once():
    cfg = bench.llama3_8b()
    attn, step = bench.step_bytes_of(cfg, 256, 4096, 16, int8=False)
    # per context token 2 (K, V) x 8 KV heads x 128 x 2 bytes; per sequence q in (fp32) + out (fp16); one id per block
    assert attn == 256 * 4096 * 4096 + 256 * 32 * 128 * 6 + 256 * 256 * 4
    layer_params = 32 * (6144 * 4096 + 4096 * 4096 + 28672 * 4096 + 4096 * 14336)
    head = 128256 * 4096
    norms = (2 * 32 + 1) * 4096
    assert step == attn * 32 + 2 * (layer_params + head + norms)
    _, step8 = bench.step_bytes_of(cfg, 256, 4096, 16, int8=True)
    assert step - step8 == layer_params  # only the layer matrices shrink to one byte per weight


def test_reference_arm_sets_its_own_thread_count_under_a_launcher():
    # a multi-process launcher exports OMP_NUM_THREADS=1 to its ranks; the CPU arm must not inherit that
    from oracle import oracle
    code = ("import os; os.environ['OMP_NUM_THREADS'] = '1'\n"
            "from oracle import oracle\n"
            "print(oracle.set_threads(), len(os.sched_getaffinity(0)))")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=120,
                       env=dict(os.environ, OMP_NUM_THREADS="1"))
    used, cores = (int(v) for v in r.stdout.split())
    assert used == cores

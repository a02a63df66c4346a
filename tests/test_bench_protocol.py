"""Host-side rules of bench.py: which workloads rotate over tensor sets, and that the GPU arm and the
reference arm describe one command line with the same `config` object (no GPU needed)."""
import json
import subprocess
import sys

import bench


def test_small_workloads_rotate_over_more_than_twice_the_l2():
    for name in ("C1", "C2"):
        cfg = bench.CONFIGS[name]
        n = bench.rotation_sets(cfg)
        assert n >= 2
        assert n * bench.tensor_bytes(cfg) >= 2 * bench.L2_BYTES
        assert (n - 1) * bench.tensor_bytes(cfg) < 2 * bench.L2_BYTES   # and no more sets than that takes


def test_large_workloads_are_timed_call_by_call():
    for name in ("C3d128", "C3d64", "C4", "C5shard", "C5"):
        cfg = bench.CONFIGS[name]
        assert bench.tensor_bytes(cfg) > bench.L2_BYTES
        assert bench.rotation_sets(cfg) == 0


def test_tensor_bytes_counts_the_nine_tensors():
    # C2: five query-shaped and four key-shaped fp16 tensors of 2 MiB each, plus 32 KiB of LSE
    assert bench.tensor_bytes(bench.CONFIGS["C2"]) == 9 * (2 << 20) + 4 * 2048 * 4


def test_both_arms_print_the_same_config_block():
    for name in ("C2", "C4"):
        cfg = bench.CONFIGS[name]
        b, desc = cfg[0], cfg[7]
        gpu_arm = bench.config_block(desc, False, b, 1, False, cfg)
        cpu_arm = bench.config_block(desc, False, b, 1, False, cfg)
        assert gpu_arm == cpu_arm
        assert ("back to back" in gpu_arm["l2"]) == (bench.rotation_sets(cfg) > 0)


def test_reference_arm_line_carries_the_contract_keys():
    out = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "1", "--warmup", "1",
                          "--config", "C1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port"
    assert line["config"] == bench.config_block(bench.CONFIGS["C1"][7], False, 1, 1, False, bench.CONFIGS["C1"])

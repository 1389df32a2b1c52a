"""Host-side logic of bench.py that needs no GPU: the work split of the long-context shape over
N ranks and the `config` object that the GPU arm and the CPU reference arm must print alike."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_strong_split_covers_every_pair_once():
    bench = load_bench()
    B, H, S, D, causal = bench.ATTN["attn_c3"]
    assert B * H == 64
    for world in (1, 2, 4, 8):
        assert (B * H) % world == 0
        cfg = bench.attention_config("attn_c3", world, "strong")
        per_rank = B * H // world
        if world > 1:
            assert f"split {per_rank} per GPU over {world} GPUs" in cfg["workload"]
            assert cfg["global_batch"] == B  # one job, not one per rank
        else:
            assert cfg["workload"].endswith("per GPU") and cfg["global_batch"] == B
        # L2 note: inputs of a rank against twice the L2
        small = 3 * per_rank * S * D * 2 <= 2 * 126e6
        assert ("input sets used in turn" in cfg["l2"]) == small
    # the weak form multiplies the batch instead
    assert bench.attention_config("attn_c3", 8, "weak")["global_batch"] == 8 * B


def test_flop_count_is_the_configured_one():
    bench = load_bench()
    assert bench.attn_flops(2, 32, 16384, 128, True) == 4.0 * 2 * 32 * 16384 * 16384 * 128 / 2
    assert abs(bench.attn_flops(2, 32, 16384, 128, True) - 4.398e12) / 4.398e12 < 1e-3
    assert bench.attn_flops(8, 12, 1024, 64, True) == 1.2884901888e10


def test_reference_arm_prints_the_gpu_arms_config():
    """`bench.py --impl reference` runs without a GPU and must describe the same workload."""
    bench = load_bench()
    for gpus in (1, 8):
        env = dict(os.environ, RANK="0")
        out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", str(gpus),
                              "--steps", "1", "--warmup", "0", "--workload", "attn_c2"],
                             capture_output=True, text=True, env=env, timeout=300)
        assert out.returncode == 0, out.stderr[-500:]
        line = json.loads(out.stdout.strip().splitlines()[-1])
        assert line["impl"] == "reference" and line["unit"] == "TFLOP/s"
        assert line["config"] == bench.attention_config("attn_c2", gpus, "weak")
        assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "port"
    # ranks other than 0 print nothing
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, env=dict(os.environ, RANK="1"), timeout=60)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_rotating_input_sets_cover_three_times_l2():
    bench = load_bench()
    l2 = 126e6
    assert bench.rotating_sets(805e6) == 1 and bench.rotating_sets(2 * l2 + 1) == 1
    for nbytes in (50.3e6, 100.7e6, 2 * l2):
        sets = bench.rotating_sets(nbytes)
        assert sets >= 2
        # between two uses of one set, the other sets alone push at least three times L2 through it
        assert (sets - 1) * nbytes >= 3 * l2
        assert (sets - 2) * nbytes < 3 * l2  # and not one set more than that needs

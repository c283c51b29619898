"""The reference arm of bench.py runs on host cores only: it must work without a GPU and print one JSON line with the
fields the measurement contract names."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["gpu_launches"] == 0


def test_config1_pairs_are_dealt_to_the_ranks_exactly_once():
    """bench.py --gpus N splits config 1 by (sequence, kv head): every pair on exactly one rank, equal shares."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    seqlens, Hk = [16384] * 4, 4
    for world in (1, 2, 4, 8, 16):
        seen = []
        for rank in range(world):
            heads, seqs = bench.shard_config1(rank, world, seqlens, Hk)
            seen += [(s, h) for h in heads for s in seqs]
        assert sorted(seen) == sorted((s, h) for s in range(4) for h in range(Hk)), world
    # the analytic count of attended pairs is additive over the shards
    whole = bench.analytic_pairs(seqlens, Hk, 2, 64, 16)
    parts = 0
    for rank in range(8):
        heads, seqs = bench.shard_config1(rank, 8, seqlens, Hk)
        parts += bench.analytic_pairs([seqlens[i] for i in seqs], len(heads), 2, 64, 16)
    assert parts == whole

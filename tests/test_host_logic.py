"""Host-side logic that needs no GPU: the sharding arithmetic (incl. a world_size-2 gloo run),
device-array views, and plan vocabulary."""
import os
import subprocess
import sys

import numpy as np
import pytest

import juliavision_b200 as jv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("total,world,align", [(1500, 8, 128), (64, 8, 1), (65536, 4, 128), (5, 8, 1), (0, 2, 4),
                                               (1000, 3, 64)])
def test_shard_ranges_partition(total, world, align):
    prev = 0
    sizes = []
    for r in range(world):
        b, e = jv.shard_range(total, world, r, align)
        assert (b, e) == jv.shard_range_py(total, world, r, align)
        assert b == prev and e >= b
        assert b % align == 0 or b == total
        prev = e
        sizes.append(e - b)
    assert prev == total
    full = [s for s in sizes if s]
    assert not full or max(full) - min(full) < 2 * align  # one whole unit, plus the ragged last unit


def test_shard_range_rejects_bad_arguments():
    with pytest.raises(jv.B200Error):
        jv.shard_range(10, 0, 0, 1)
    with pytest.raises(jv.B200Error):
        jv.shard_range(10, 2, 2, 1)


def test_device_array_views_are_stride_arithmetic():
    a = jv.DeviceArray(None, 4096, np.float16, (64, 20, 1500, 1))       # (E,H,L,B) projection output
    q = a.permute((0, 2, 1, 3))                                        # (E,L,H,B) view
    assert q.shape == (64, 1500, 20, 1) and q.strides == (1, 1280, 64, 1280 * 1500)
    assert not q.isdense() and a.isdense()
    s = a.slice(2, 10, 20)
    assert s.ptr == 4096 + 10 * 1280 * 2 and s.shape[2] == 10
    with pytest.raises(ValueError):
        q.reshape(64 * 1500, 20)
    assert a.reshape(1280, 1500).strides == (1, 1280)


def test_gather_shards_gloo_world2(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(
        "import os, sys, torch, torch.distributed as dist\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "from juliavision_b200.shard import shard_range_py, gather_shards\n"
        "dist.init_process_group('gloo')\n"
        "r, w = dist.get_rank(), dist.get_world_size()\n"
        "full = torch.arange(37 * 3, dtype=torch.float32).reshape(37, 3)\n"
        "b, e = shard_range_py(37, w, r, 8)\n"
        "got = gather_shards(full[b:e].clone(), 37, w, 8)\n"
        "assert torch.equal(got, full), (r, got.shape)\n"
        "dist.barrier(); dist.destroy_process_group(); print('ok', r)\n")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                         capture_output=True, text=True, timeout=240, env=env)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count("ok") == 2


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: one JSON line with the contract's keys, timed on the
    oracle (the CPU form of the path), marked as the reference arm."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for k in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert k in line, k
    assert line["impl"] == "reference" and line["metric"] == "encoder_ms_per_img" and line["higher_is_better"] is False
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0

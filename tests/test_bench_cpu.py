"""bench.py's reference arm runs on the host alone: its JSON line must carry the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "clip_fwd_bwd_tflops" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert abs(d["cpu_baseline"]["value"] - d["value"]) < 1e-9
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["config"]["workload"] == "clip_b32768_d1152_bf16"


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert out.returncode == 0
    assert not [l for l in out.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_samples_rows_only_when_the_step_is_too_large():
    sys.path.insert(0, ROOT)
    import bench
    # the headline configuration is timed whole; the ring configurations as a row sample against all columns
    assert bench.cpu_sample_rows(32768, 1152, 1.2e13) == 32768
    rows = bench.cpu_sample_rows(262144, 1024, 1.2e13)
    assert 512 <= rows < 262144 and rows % 512 == 0
    assert 8.0 * rows * 262144 * 1024 <= 1.2e13


def test_blocked_cpu_step_is_the_dense_loss():
    """The reference arm's workload (oracle.dense.clip_blocked_step) is the same loss and the same gradients
    as the dense formulation; a row sample does the full problem's work per row."""
    import torch
    import torch.nn.functional as F
    from oracle import dense
    g = torch.Generator().manual_seed(5)
    x = F.normalize(torch.randn(700, 48, generator=g), dim=1)
    y = F.normalize(torch.randn(700, 48, generator=g), dim=1)
    loss, dx, dy = dense.clip_blocked_step(x, y, 0.07, row_block=256)
    rl, rx, ry = dense.clip_dense(x, y, 0.07, True)
    dense.assert_parity(float(loss), rl, (dx, dy), (rx, ry), "blocked cpu step")
    _l, dxs, dys = dense.clip_blocked_step(x, y, 0.07, row_block=128, rows=256)
    assert dxs.shape == (256, 48) and dys.shape == (700, 48)

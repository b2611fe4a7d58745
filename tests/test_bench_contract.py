"""The command-line contract of bench.py that does not need a GPU: defaults, and the reference arm's answer."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-500:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference"
    assert ("unavailable" in rec and rec["unavailable"]) or "value" in rec


def test_argument_defaults_finish_quickly():
    sys.path.insert(0, ROOT)
    import bench
    old = sys.argv
    sys.argv = ["bench.py"]
    try:
        a = bench.parse_args()
    finally:
        sys.argv = old
    assert a.gpus == 1 and a.warmup >= 3 and 1 <= a.steps <= 10 and a.impl == "oslo_b200" and a.mode == "train"
    assert a.model == "gptj-6b" and a.seq == 2048


def _reference_installed() -> bool:
    return os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "oslo"))


def _reference_ranks(rank, world, out_dir):
    """The reference arm's training loop on CPU ranks (gloo): the unmodified reference package builds the model,
    torch DDP over its data-parallel group reduces the gradients, every rank ends with the same weights."""
    import types
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from baseline import reference_runner as rr
    assert rr.probe() == ""
    args = types.SimpleNamespace(gpus=world, steps=2, warmup=1, model="gptj-tiny", seq=16, batch_per_gpu=4,
                                 no_e2e=False, mode="train")
    line = rr.run_train(args, None, force_cpu=True)
    assert line["impl"] == "reference" and line["n_gpus"] == world and line["value"] > 0
    assert line["config"]["global_batch"] == 4 * world and line["e2e"]["h2d_bytes_per_step"] == 4 * 16 * 8
    assert 2.0 < line["e2e"]["last_loss"] < 5.5          # ln(128) = 4.85 at random init, falling
    assert "oslo_b200" not in sys.modules                # nothing of this framework is on the reference's path
    if rank == 0:
        with open(os.path.join(out_dir, "line.json"), "w") as f:
            json.dump(line, f)


def test_reference_arm_trains_the_unmodified_reference_on_cpu_ranks(tmp_path):
    import pytest
    if not _reference_installed():
        pytest.skip("reference package not installed under baseline/_ref")
    from tests.dist_utils import run_distributed
    run_distributed(_reference_ranks, 2, str(tmp_path), fresh=True)
    rec = json.load(open(tmp_path / "line.json"))
    assert rec["config"]["parallelism"].startswith("dp2") and rec["steps"] == 2 and rec["warmup"] == 1


def _reference_decode_rank(rank, world, out_dir):
    import types
    sys.path.insert(0, ROOT)
    from baseline import reference_runner as rr
    assert rr.probe() == ""
    args = types.SimpleNamespace(gpus=world, steps=1, warmup=1, model="gptj-tiny", no_e2e=False, mode="decode",
                                 prompt=8, new_tokens=6, decode_batch=2, tp=1)
    line = rr.run_decode(args, None, force_cpu=True)
    assert line["impl"] == "reference" and line["unit"] == "ms/token" and line["higher_is_better"] is False
    assert line["value"] > 0 and line["e2e"]["d2h_bytes_per_step"] == 2 * 14 * 8
    assert "oslo_b200" not in sys.modules


def test_reference_arm_greedy_decode_runs_the_unmodified_reference_on_cpu(tmp_path):
    """The reference's own ``generate()`` (greedy search, its vendored 4.x loop) runs on the installed stack."""
    import pytest
    if not _reference_installed():
        pytest.skip("reference package not installed under baseline/_ref")
    from tests.dist_utils import run_distributed
    run_distributed(_reference_decode_rank, 1, str(tmp_path), fresh=True)


def test_default_plan_follows_the_model_parallel_sweep():
    sys.path.insert(0, ROOT)
    import bench
    names = {n: bench.default_plan(n) for n in (1, 2, 4, 8)}
    assert names[1][0]["name"] == "single" and names[1][1] == []
    assert (names[2][0]["tp"], names[2][0]["pp"]) == (2, 1) and names[2][1][0]["name"] == "dp2_zero1"
    assert (names[4][0]["tp"], names[4][0]["pp"]) == (4, 1)
    p8, also8 = names[8]
    assert (p8["tp"], p8["pp"], p8["micro"]) == (2, 4, 4)          # 64 sequences as 16 micro-batches of 4
    assert [a["name"] for a in also8] == ["dp8_zero1", "tp8_b8x2048", "gptneo1.3b_tp2xpp2xdp2"]
    assert also8[1]["replica_batch"] == 8
    neo = also8[2]       # GPT-Neo 1.3B: 2 replicas of tp2 x pp2, 8 micro-batches of 4 sequences per replica and step
    assert neo["model"] == "gpt-neo-1.3b" and 8 // (neo["tp"] * neo["pp"]) == 2 and neo["replica_batch"] // neo["micro"] == 8


def test_fusion_mode_times_generate_before_and_after_fuse():
    """``--mode fusion`` (the reference's tests/gpt2/gpt2_test_kernel_fusion.py as a benchmark) at a debug size on CPU:
    one JSON line, time-like metric, the three timings; the reference arm says why it cannot run this mode here."""
    env = dict(os.environ, OSLO_B200_BACKEND="gloo")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--mode", "fusion", "--layers", "1",
                        "--new-tokens", "6", "--steps", "1", "--warmup", "1"], capture_output=True, text=True,
                       timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stderr[-800:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["higher_is_better"] is False and rec["unit"] == "s" and rec["metric"].endswith("(debug)")
    assert rec["value"] == rec["after_fuse_s"] > 0 and rec["before_fuse_s"] > 0 and rec["after_fuse_fused_ngram_s"] > 0
    assert rec["vs_baseline"] is None and rec["config"]["num_beams"] == 5 and rec["config"]["no_repeat_ngram_size"] == 4
    sys.path.insert(0, ROOT)
    import bench
    assert bench.FUSION_PUBLISHED[4]["after_fuse_s"] == 3.859266519546509
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--mode", "fusion"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0
    rec = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][0])
    assert rec["impl"] == "reference" and rec["unavailable"]

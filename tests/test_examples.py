"""The example scripts run end to end on CPU ranks: preprocess a corpus, train TP2 x PP2 (and DP2 with ZeRO-1),
interrupt, resume to the same weights, merge, generate from the merged checkpoint."""
import json
import os
import socket
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "examples")


def _port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(cmd, **env):
    e = dict(os.environ, OSLO_B200_BACKEND="gloo", OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="", **env)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env=e)
    assert r.returncode == 0, (cmd, r.stdout[-1500:], r.stderr[-3000:])
    return r


def _torchrun(n, script, *args):
    return _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                 "--master-addr", "127.0.0.1", "--master-port", str(_port()), os.path.join(EX, script), *args])


def test_preprocess_train_resume_merge_generate(tmp_path):
    corpus = tmp_path / "corpus.jsonl"
    with open(corpus, "w") as f:
        for i in range(200):
            f.write(json.dumps({"text": f"document {i}: " + "the quick brown fox jumps over the lazy dog. " * (1 + i % 5)}) + "\n")
    data = str(tmp_path / "data" / "corpus")
    out = _run([sys.executable, os.path.join(EX, "preprocess.py"), "--input", str(corpus), "--output", data])
    assert "200 documents" in out.stdout and os.path.isfile(data + ".bin") and os.path.isfile(data + ".idx")

    common = ["--model", "gptj", "--tiny", "--tp", "2", "--pp", "2", "--batch-size", "4", "--micro-batch-size", "2",
              "--seq", "32", "--data", data, "--lr", "1e-3"]
    full, part = str(tmp_path / "full"), str(tmp_path / "part")
    _torchrun(4, "train.py", *common, "--steps", "4", "--save", full, "--merge", "--metrics", str(tmp_path / "m.jsonl"))
    recs = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert [r["step"] for r in recs] == [1, 2, 3, 4] and recs[-1]["loss"] < recs[0]["loss"]
    for tp in range(2):
        for pp in range(2):
            assert os.path.isfile(os.path.join(full, f"pytorch_model_tp={tp}_pp={pp}.bin"))
            assert os.path.isfile(os.path.join(full, f"oslo_state_tp={tp}_pp={pp}_dp=0.pt"))

    # 2 steps, stop, resume for 2 more: the same weights as 4 uninterrupted steps
    _torchrun(4, "train.py", *common, "--steps", "2", "--save", part)
    _torchrun(4, "train.py", *common, "--steps", "4", "--save", part, "--resume", "--merge")
    a = torch.load(os.path.join(full, "merged", "pytorch_model.bin"), weights_only=True)
    b = torch.load(os.path.join(part, "merged", "pytorch_model.bin"), weights_only=True)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k

    # the split files of the first run, merged by the stand-alone script, give the same file as --merge did; the script
    # also checks the merged model's logits against the parallel model's
    again = str(tmp_path / "again")
    out = _torchrun(4, "merge.py", "--model", "gptj", "--checkpoint", full, "--tp", "2", "--pp", "2", "--output", again,
                    "--check")
    assert "logit difference" in out.stdout
    m = torch.load(os.path.join(again, "pytorch_model.bin"), weights_only=True)
    assert m.keys() == a.keys() and all(torch.equal(m[k], a[k]) for k in a)

    # the 4 blocks split 3 + 1 over the two stages instead of 2 + 2: where the stage boundary lies does not change
    # the result (up to the summation order of the gradient norm over the ranks)
    uneven = str(tmp_path / "uneven")
    _torchrun(4, "train.py", *common, "--pipeline-partition", "balanced", "--steps", "4", "--save", uneven, "--merge")
    c = torch.load(os.path.join(uneven, "merged", "pytorch_model.bin"), weights_only=True)
    assert a.keys() == c.keys()
    for k in a:
        assert torch.allclose(a[k], c[k], atol=1e-5, rtol=1e-4), k

    gen = _run([sys.executable, os.path.join(EX, "generate.py"), "--model", "gptj", "--checkpoint",
                os.path.join(full, "merged"), "--prompt", "the quick", "--max-new-tokens", "8", "--num-beams", "2"])
    assert gen.stdout.startswith("the quick") and "8 new tokens" in gen.stderr


def test_train_example_data_parallel_zero1(tmp_path):
    out = str(tmp_path / "dp")
    _torchrun(2, "train.py", "--model", "gpt2", "--tiny", "--batch-size", "4", "--micro-batch-size", "2", "--seq", "16",
              "--steps", "2", "--save", out, "--watchdog")
    assert os.path.isfile(os.path.join(out, "pytorch_model.bin"))      # no model parallelism: the plain HF file
    assert all(os.path.isfile(os.path.join(out, f"oslo_state_tp=0_pp=0_dp={d}.pt")) for d in range(2))


def test_training_restarts_itself_from_the_last_complete_checkpoint(tmp_path):
    """Elastic recovery with a host-side fault: the last rank raises at step 5 of 6 during the first launch attempt;
    ``torchrun --max-restarts 1`` launches the workers again, ``--auto-resume`` finds the generation of step 4 and the
    run ends with exactly the weights of an uninterrupted run. A generation whose shard was damaged afterwards is
    skipped by all ranks together."""
    common = ["--model", "gptj", "--tiny", "--tp", "2", "--batch-size", "4", "--micro-batch-size", "2", "--seq", "16",
              "--lr", "1e-3", "--steps", "6", "--save-every", "2", "--auto-resume"]
    straight, broken = str(tmp_path / "straight"), str(tmp_path / "broken")
    _torchrun(2, "train.py", *common, "--save", straight)
    r = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--max-restarts=1",
              "--master-addr", "127.0.0.1", "--master-port", str(_port()), os.path.join(EX, "train.py"), *common,
              "--save", broken, "--fail-at-step", "5"])
    assert "injected failure at step 5" in r.stderr and "resumed from" in r.stderr and "step-00000004" in r.stderr
    for tp in range(2):
        a = torch.load(os.path.join(straight, f"pytorch_model_tp={tp}_pp=0.bin"), weights_only=True)
        b = torch.load(os.path.join(broken, f"pytorch_model_tp={tp}_pp=0.bin"), weights_only=True)
        assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    gens = sorted(os.listdir(os.path.join(broken, "checkpoints")))
    assert gens == ["latest", "step-00000004", "step-00000006"]          # --keep 2
    assert open(os.path.join(broken, "checkpoints", "latest")).read().strip() == "step-00000006"

    # damage one shard of the newest generation: every rank falls back to step 4 (and trains on to step 8)
    victim = os.path.join(broken, "checkpoints", "step-00000006", "pytorch_model_tp=1_pp=0.bin")
    with open(victim, "r+b") as f:
        f.truncate(os.path.getsize(victim) // 2)
    more = [("8" if x == "6" else x) for x in common]
    r = _torchrun(2, "train.py", *more, "--save", broken)
    assert "step-00000004" in r.stderr and "resumed from" in r.stderr
    assert open(os.path.join(broken, "checkpoints", "latest")).read().strip() == "step-00000008"


def test_preprocess_example_converts_a_directory_tree_and_continues_after_an_interruption(tmp_path):
    src = tmp_path / "corpora"
    (src / "a").mkdir(parents=True)
    (src / "b").mkdir()
    with open(src / "a" / "big.jsonl", "w") as f:
        for i in range(30):
            f.write(json.dumps({"text": f"document number {i} of the big file"}) + "\n")
    with open(src / "b" / "small.txt", "w") as f:
        f.write("first document\n\nsecond document\n")
    out = tmp_path / "data"
    cmd = [sys.executable, os.path.join(EX, "preprocess.py"), "--input-dir", str(src), "--output", str(out), "--small-first"]
    r = _run(cmd)
    lines = [l for l in r.stdout.splitlines() if ".bin/.idx" in l]
    assert "small" in lines[0] and "2 documents" in lines[0] and "30 documents" in lines[1]      # smallest file first
    assert open(out / "done.txt").read().split() == [os.path.join("b", "small.txt"), os.path.join("a", "big.jsonl")]
    from oslo_b200.data import MMapIndexedDataset
    assert len(MMapIndexedDataset(str(out / "a" / "big"))) == 30 and len(MMapIndexedDataset(str(out / "b" / "small"))) == 2
    # a batch that was interrupted after the first file: only the second is converted now
    os.remove(out / "a" / "big.bin")
    os.remove(out / "a" / "big.idx")
    with open(out / "done.txt", "w") as f:
        f.write(os.path.join("b", "small.txt") + "\n")
    r = _run(cmd)
    assert "already converted" in r.stdout and os.path.isfile(out / "a" / "big.bin")

"""The decode step gives the same bits whether its kernels are launched as programmatic dependents of one
another (the default: a kernel's blocks may be placed while the kernel before drains and hold at
griddepcontrol.wait) or the ordinary, fully serialised way (B200_SERIAL_LAUNCH=1).

The switch is read once per process, so each mode runs in a process of its own: a tiny random-init engine
serves two prompts through B200Backend (prompt passes, then decode steps from the captured CUDA graph) and
prints its tokens and a checksum of the logits of every step.  An overlap that let a kernel read what the kernel
before had not finished writing would show as different bits here."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

SCRIPT = r"""
import importlib, json, sys
import torch
sys.path.insert(0, sys.argv[1])
eng_mod = importlib.import_module("inference-server_b200.engine")
backend_mod = importlib.import_module("inference-server_b200.backend")
engine = eng_mod.DecodeEngine(eng_mod.CONFIGS["tiny"], num_blocks=96, max_batch=4, max_pages_per_seq=16, device="cuda",
                              seed=11, keep_logits=True)
backend = backend_mod.B200Backend(engine, max_new_tokens=24)
g = torch.Generator().manual_seed(3)
batch, toks, sums = None, [], []
for i, n in enumerate((53, 17, 90)):
    kv, first, m = backend.prefill(torch.randint(0, 4096, (n,), generator=g).tolist(), f"s{i}")
    batch = backend.splice_into_batched(batch, kv, m)
    toks.append(first)
cur = torch.tensor(toks).view(-1, 1)
trace = [toks]
for step in range(16):
    nxt, batch = backend.decode_step_batched(cur, batch, None, None)
    trace.append(nxt.tolist())
    sums.append(engine.last_logits.view(torch.int16).to(torch.int64).sum().item())  # bit pattern of the bf16 logits
    cur = nxt.view(-1, 1)
engine.check_status("launch modes")
print("RESULT " + json.dumps({"tokens": trace, "logit_bits": sums}))
"""


def run_mode(serial: str) -> dict:
    env = dict(os.environ)
    env["B200_SERIAL_LAUNCH"] = serial
    out = subprocess.run([sys.executable, "-c", SCRIPT, ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_overlapped_and_serial_launches_give_the_same_bits():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    overlapped = run_mode("0")
    serial = run_mode("1")
    assert overlapped["tokens"] == serial["tokens"]
    assert overlapped["logit_bits"] == serial["logit_bits"]
    assert len(overlapped["tokens"]) == 17 and len(overlapped["logit_bits"]) == 16


def test_prompt_attention_parity_also_holds_for_the_mma_sync_kernel_at_head_dim_128():
    """head_dim 128 takes the tcgen05 kernel by default, so the parity tests of the prompt attention exercise the
    mma.sync kernel only at head_dim 64; with B200_PREFILL_MMA_SYNC=1 (read once per process) the same tests run
    the mma.sync kernel at every shape."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    env = dict(os.environ)
    env["B200_PREFILL_MMA_SYNC"] = "1"
    out = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_prefill_attn.py"), "-x", "-q",
                          "-m", "gpu", "-p", "no:cacheprovider"], env=env, cwd=ROOT, capture_output=True, text=True,
                         timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-1000:]
    assert " passed" in out.stdout and "failed" not in out.stdout

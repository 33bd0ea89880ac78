"""Host-side pieces of bench.py that need no GPU."""
import importlib.util
import os

import numpy as np

from conftest import ROOT


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_prompt_lengths_are_dealt_to_ranks_by_context_load():
    bench = load_bench()
    world, batch = 8, 256
    lens = np.random.default_rng(12345).integers(512, 4097, size=world * batch).tolist()
    shares = [bench.balanced_share(lens, world, r, batch) for r in range(world)]
    assert all(len(s) == batch for s in shares)
    assert sorted(x for s in shares for x in s) == sorted(lens)  # every sequence goes to exactly one rank
    sums = [sum(s) for s in shares]
    assert max(sums) / min(sums) < 1.001
    # the workload builder gives a rank its share, shuffled, with a block table that fits it
    cfg = bench.pkg("engine").CONFIGS["qwen3-30b-a3b"]
    mine, table, blocks, max_pages = bench.build_workload(cfg, batch, 256, seed=3, world=world, rank=3, balance=True)
    assert sorted(mine) == sorted(shares[3])
    pages = [(n + 256 + 15) // 16 for n in mine]
    assert table.shape == (batch, max(pages)) and blocks >= sum(pages)
    own, *_ = bench.build_workload(cfg, batch, 256, seed=3, world=world, rank=3, balance=False)
    assert own != mine and len(own) == batch

"""The unchanged HuggingFace Qwen3-MoE forward (what the reference's TorchBackend calls) running on this
package's kernels through the attention / experts / cache hooks (B200)."""
import pytest
import torch

from conftest import pkg, rel_err
from oracle.ref_decode import hf_config

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_hf_forward_with_plugins_matches_the_engine_step(ops):
    from transformers import Qwen3MoeForCausalLM

    eng_mod, plugins = pkg("engine"), pkg("hf_plugins")
    plugins.register()
    torch.manual_seed(0)
    cfg = hf_config(eng_mod.CONFIGS["tiny"], attn_implementation="eager", experts_implementation="eager")
    model = Qwen3MoeForCausalLM(cfg).float().eval()
    engine = eng_mod.engine_from_hf(model, num_blocks=64, max_batch=4, max_pages_per_seq=8, device=DEV, keep_logits=True)
    g = torch.Generator().manual_seed(2)
    lens = [37, 64, 90, 5]
    table = torch.arange(32, dtype=torch.int32).view(4, 8)
    for b, n in enumerate(lens):
        engine.prefill(torch.randint(0, 4096, (n,), generator=g).tolist(), table[b].tolist())
    cur = torch.randint(0, 4096, (4,), generator=g)
    # page pools as they are before the step: the HF run gets its own copy, the engine runs on the originals
    k2 = [p.clone() for p in engine.k_pools]
    v2 = [p.clone() for p in engine.v_pools]

    engine.block_table.copy_(table)
    engine.ctx_lens.copy_(torch.tensor(lens, dtype=torch.int32))
    engine.tokens.copy_(cur)
    nxt = engine.step(4).clone()
    ref_logits = engine.last_logits.float().clone()

    gm = model.to(DEV).to(torch.bfloat16)
    gm.config._attn_implementation = "b200_paged"
    gm.config._experts_implementation = "b200_fp8"
    cache = plugins.PagedKVCache(k2, v2, table.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV))
    with torch.no_grad():
        out = gm(cur.to(DEV).view(4, 1), position_ids=torch.tensor(lens, device=DEV).view(4, 1),
                 past_key_values=cache, use_cache=True, b200_cache=cache)
    cache.advance()
    ops.read_status(cache.status, "kv_append via PagedKVCache")
    logits = out.logits[:, -1, :].float()
    assert rel_err(logits, ref_logits) < 3e-2  # same kernels for attention and experts; glue differs (torch vs fused)
    assert (logits.argmax(-1) == nxt).sum() >= 3
    # both paths appended this step's K rows to the same page slots (the engine's graph warm-up also touches
    # later slots, so only the slot of this step is compared)
    for a, b in zip(k2, engine.k_pools):
        for row, n in enumerate(lens):
            page, slot = int(table[row, n // 16]), n % 16
            # 128 bf16 values after two layers of torch-vs-fused glue; the engine also routes on fp32 router logits
            # while the HF module's gate produces bf16 ones, so a near-tied expert may differ for a token
            assert rel_err(a[page, :, slot, :], b[page, :, slot, :]) < 1e-1
    assert cache.positions.tolist() == [n + 1 for n in lens]

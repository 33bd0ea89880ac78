"""Paged decode engine: one Qwen3-MoE-shaped decode step on block tables.

This is the model-forward side of the reference's hot entry
``TorchBackend.decode_step_batched``
(src/inference_server/backends/torch_backend.py:305-322), rebuilt so that a
step reads the KV page pools in place instead of a dense left-padded cache:

  per layer   fused q/k/v projection (``b200_dense_gemm_bf16``)
              -> ``b200_qk_norm_rope_append`` (per-head q/k RMSNorm, RoPE, page write)
              -> ``b200_paged_attn_decode`` -> o projection (``b200_dense_gemm_bf16``)
              -> ``b200_add_rmsnorm`` (residual + RMSNorm) -> router projection (``b200_dense_gemm_bf16``)
              -> ``b200_moe_fp8_forward_add_rmsnorm`` (route, permute+quantise, two
                 grouped GEMMs, combine + residual + the next layer's input norm)
  final       ``b200_lm_head_argmax`` (lm_head with the arg-max over the vocabulary in its epilogue)

Every kernel of the step is this package's own: the element-wise glue, paged attention, the FP8 MoE layer and
the dense bf16 projections (tcgen05); the one library call left is the embedding row gather.  The whole step is
captured once per batch size in a CUDA graph; block table, context lengths and input tokens live in static
device buffers that the graph reads.

Pools use the reference layout [num_blocks, n_kv_heads, 16, head_dim] per layer
(src/inference_server/kv_cache/block_manager.py:33-49) and can be the very
tensors a reference ``BlockManager`` allocated.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import ops, quant

PAGE = 16


@dataclass(frozen=True)
class ModelConfig:
    name: str
    vocab_size: int
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    experts: int
    top_k: int
    moe_inter: int
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    norm_topk_prob: bool = True


CONFIGS = {
    # BASELINE config 4: Qwen3-30B-A3B shape
    "qwen3-30b-a3b": ModelConfig("qwen3-30b-a3b", 151936, 2048, 48, 32, 4, 128, 128, 8, 768),
    # BASELINE config 5: Qwen3-235B-A22B shape (needs expert parallelism to fit)
    "qwen3-235b-a22b": ModelConfig("qwen3-235b-a22b", 151936, 4096, 94, 64, 4, 128, 128, 8, 1536),
    # BASELINE config 1: the tiny parity model
    "tiny": ModelConfig("tiny", 4096, 512, 2, 8, 2, 64, 16, 4, 256),
}


class LayerWeights:
    """Weights of one decoder layer, already in their run-time formats."""

    __slots__ = ("ln1", "wqkv", "q_norm", "k_norm", "wo", "ln2", "router", "w13", "w13_scale", "w2", "w2_scale")


def rope_tables(head_dim: int, theta: float, max_pos: int, device, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def random_layer(cfg: ModelConfig, device, gen: torch.Generator, std: float = 0.02,
                 local_experts: int | None = None) -> LayerWeights:
    """Random-init weights (N(0, std)), experts quantised to e4m3 128x128 blocks on the device.
    With `local_experts` only that many experts are created (this rank's shard under expert parallelism)."""
    H, D = cfg.hidden, cfg.head_dim
    w = LayerWeights()
    bf = torch.bfloat16

    def rn(*shape):
        return torch.randn(*shape, device=device, generator=gen, dtype=torch.float32) * std

    w.ln1 = torch.ones(H, device=device, dtype=bf)
    w.ln2 = torch.ones(H, device=device, dtype=bf)
    w.q_norm = torch.ones(D, device=device, dtype=bf)
    w.k_norm = torch.ones(D, device=device, dtype=bf)
    w.wqkv = rn((cfg.q_heads + 2 * cfg.kv_heads) * D, H).to(bf)
    w.wo = rn(H, cfg.q_heads * D).to(bf)
    w.router = rn(cfg.experts, H).to(bf)
    n_exp = local_experts or cfg.experts
    w.w13, w.w13_scale = quant.quantize_weight_blocks(rn(n_exp, 2 * cfg.moe_inter, H))
    w.w2, w.w2_scale = quant.quantize_weight_blocks(rn(n_exp, H, cfg.moe_inter))
    w.w13, w.w2 = quant.tile_weight_blocks(w.w13), quant.tile_weight_blocks(w.w2)
    return w


def layer_from_hf(layer, device) -> LayerWeights:
    """Run-time weights of one ``Qwen3MoeDecoderLayer`` (the model class the reference loads for a
    Qwen3-MoE checkpoint): projections in bf16, q/k/v fused, experts quantised to e4m3 128x128 blocks."""
    bf = torch.bfloat16
    at, mlp = layer.self_attn, layer.mlp
    w = LayerWeights()

    def dev(t):
        return t.detach().to(device=device, dtype=bf).contiguous()

    w.ln1, w.ln2 = dev(layer.input_layernorm.weight), dev(layer.post_attention_layernorm.weight)
    w.q_norm, w.k_norm = dev(at.q_norm.weight), dev(at.k_norm.weight)
    w.wqkv = dev(torch.cat([at.q_proj.weight, at.k_proj.weight, at.v_proj.weight], dim=0))
    w.wo = dev(at.o_proj.weight)
    w.router = dev(mlp.gate.weight)
    w.w13, w.w13_scale = quant.quantize_weight_blocks(mlp.experts.gate_up_proj.detach().to(device).float())
    w.w2, w.w2_scale = quant.quantize_weight_blocks(mlp.experts.down_proj.detach().to(device).float())
    w.w13, w.w2 = quant.tile_weight_blocks(w.w13), quant.tile_weight_blocks(w.w2)
    return w


def engine_from_hf(model, num_blocks: int, max_batch: int, max_pages_per_seq: int, device="cuda", **kw):
    """DecodeEngine holding the weights of a transformers ``Qwen3MoeForCausalLM``."""
    c = model.config
    cfg = ModelConfig("from-hf", c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads,
                      c.num_key_value_heads, c.head_dim, c.num_experts, c.num_experts_per_tok,
                      c.moe_intermediate_size, float(c.rope_parameters["rope_theta"]), c.rms_norm_eps,
                      bool(c.norm_topk_prob))
    bf = torch.bfloat16
    layers = [layer_from_hf(lyr, device) for lyr in model.model.layers]
    return DecodeEngine(cfg, num_blocks, max_batch, max_pages_per_seq, device=device, layers=layers,
                        embed=model.model.embed_tokens.weight.detach().to(device=device, dtype=bf).contiguous(),
                        lm_head=model.lm_head.weight.detach().to(device=device, dtype=bf).contiguous(),
                        final_norm=model.model.norm.weight.detach().to(device=device, dtype=bf).contiguous(), **kw)


class DecodeEngine:
    """Owns weights, KV page pools and the per-batch-size CUDA graphs of the decode step."""

    def __init__(self, cfg: ModelConfig, num_blocks: int, max_batch: int, max_pages_per_seq: int,
                 device: str | torch.device = "cuda", seed: int = 0, layers: list[LayerWeights] | None = None,
                 embed: torch.Tensor | None = None, lm_head: torch.Tensor | None = None,
                 final_norm: torch.Tensor | None = None, k_pools=None, v_pools=None, use_graphs: bool = True,
                 split_tokens: int | None = None, ep_group=None, ep_capacity: int | None = None,
                 ep_transport: str = "p2p", graph_buckets: bool = True, keep_logits: bool = False):
        if not torch.cuda.is_available():
            raise RuntimeError("DecodeEngine needs a CUDA device; this path has no CPU implementation")
        self.cfg = cfg
        self.device = torch.device(device)
        # The step picks its next tokens inside the lm_head kernel and never writes the [batch, vocab] logits.
        # With keep_logits they are computed as well, by a second pass over lm_head, into `last_logits` (for
        # tests and inspection; set before the first step, the graphs are captured with or without it).
        self.keep_logits = keep_logits
        self.last_logits = None
        self.max_batch = max_batch
        self.max_pages = max_pages_per_seq
        self.num_blocks = num_blocks
        self.use_graphs = use_graphs
        bf = torch.bfloat16
        gen = torch.Generator(device=self.device).manual_seed(seed)
        # expert parallelism: this rank owns experts [rank * E / W, (rank + 1) * E / W) of every layer
        self.ep_group = ep_group
        self.ep_world = 1
        if ep_group is not None:
            import torch.distributed as dist
            self.ep_world = dist.get_world_size(ep_group)
            if cfg.experts % self.ep_world:
                raise ValueError(f"{cfg.experts} experts do not divide over {self.ep_world} ranks")
        local = cfg.experts // self.ep_world if self.ep_world > 1 else None
        self.layers = layers if layers is not None else [random_layer(cfg, self.device, gen, local_experts=local)
                                                         for _ in range(cfg.layers)]
        std = 0.02
        self.embed = embed if embed is not None else (
            torch.randn(cfg.vocab_size, cfg.hidden, device=self.device, generator=gen) * std).to(bf)
        self.lm_head = lm_head if lm_head is not None else (
            torch.randn(cfg.vocab_size, cfg.hidden, device=self.device, generator=gen) * std).to(bf)
        self.final_norm = final_norm if final_norm is not None else torch.ones(cfg.hidden, device=self.device, dtype=bf)
        # Pools the engine allocates itself get one block more than the caller may hand out: the scratch page
        # that the padding rows of a bucketed CUDA graph write their K/V to (see step).  Pools given from outside
        # (a reference BlockManager's) have no such page; graphs are then captured per exact batch size, and an
        # expert-parallel engine (whose exchange always runs at the full shape) can only step at its full batch.
        own_pools = k_pools is None and v_pools is None
        self.scratch_block = num_blocks if (own_pools and graph_buckets) else None
        shape = (num_blocks + (1 if self.scratch_block is not None else 0), cfg.kv_heads, PAGE, cfg.head_dim)
        self.k_pools = k_pools if k_pools is not None else [torch.zeros(shape, device=self.device, dtype=bf) for _ in range(cfg.layers)]
        self.v_pools = v_pools if v_pools is not None else [torch.zeros(shape, device=self.device, dtype=bf) for _ in range(cfg.layers)]
        self.cos, self.sin = rope_tables(cfg.head_dim, cfg.rope_theta, max_pages_per_seq * PAGE, self.device, bf)
        self.scale = cfg.head_dim ** -0.5
        self._fixed_split = split_tokens
        self.split_tokens = split_tokens or ops.default_split_tokens(max_batch, cfg.kv_heads, max_pages_per_seq * PAGE)

        # static step state (read by the captured graphs)
        self.tokens = torch.zeros(max_batch, dtype=torch.int64, device=self.device)
        self.ctx_lens = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.block_table = torch.zeros(max_batch, max_pages_per_seq, dtype=torch.int32, device=self.device)
        self.next_tokens = torch.zeros(max_batch, dtype=torch.int64, device=self.device)
        self.attn_ws = ops.paged_attn_workspace(max_batch, cfg.q_heads, cfg.head_dim, max_pages_per_seq, PAGE,
                                                self.split_tokens, self.device)
        self.moe_ws = ops.moe_fp8_workspace(max_batch, cfg.experts, cfg.top_k, cfg.hidden, cfg.moe_inter, self.device)
        self.gemm_status = torch.zeros(64, dtype=torch.int32, device=self.device)  # dense projections, lm_head
        self._fused_router = ops.add_rmsnorm_route_supported(cfg.hidden, cfg.experts, cfg.top_k)
        self._fused_qkv = ops.qkv_rope_append_supported(cfg.head_dim, cfg.hidden)
        widest = max((cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim, cfg.hidden, cfg.experts)
        self.gemm_ws = ops.dense_gemm_workspace(min(max_batch, 256), widest, self.device)  # K-split partial tiles
        self.argmax_ws = ops.lm_head_argmax_workspace(self.device)
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        # rows of the current pass that are real (expert parallelism only): the router gives the rows beyond
        # it no expert, so they send nothing and receive nothing
        self.n_valid = torch.zeros(1, dtype=torch.int32, device=self.device)
        # attention split size and workspace per graph size: few rows want short splits (enough CTAs to fill the
        # GPU), a full batch long ones; the full batch's pair is (split_tokens, attn_ws)
        self._attn_by_rows: dict[int, tuple[int, torch.Tensor]] = {max_batch: (self.split_tokens, self.attn_ws)}
        self.ep_state = None
        if self.ep_world > 1:
            from . import ep
            cap = ep_capacity or ep.default_capacity(max_batch, cfg.top_k, self.ep_world)
            if ep_transport not in ("nccl", "p2p"):
                raise ValueError(f"ep_transport must be 'nccl' or 'p2p', got {ep_transport!r}")
            arena = None
            if ep_transport == "p2p":
                # receive buffers of every rank mapped into every process of the node (CUDA IPC): rows then
                # move by stores from the dispatch kernel and the down-GEMM epilogue, not by a collective.
                # Where the mapping cannot be made, every rank alike takes the NCCL transport and says so.
                arena = ep.PeerArena(cfg.hidden, self.ep_world, cap, self.device)
                if not arena.connect(ops, ep_group):
                    import warnings
                    warnings.warn("peer-memory expert parallelism unavailable, using NCCL all-to-all: "
                                  + "; ".join(arena.failures))
                    arena, ep_transport = None, "nccl"
            self.ep_arena = arena
            self.ep_transport = ep_transport
            self.ep_state = ep.EPState(max_batch, cfg.hidden, cfg.top_k, cfg.experts, self.ep_world, cap, self.device,
                                       ep_group, arena=arena)
        # Expert parallelism: every rank must run the same number of exchange passes.  `round_hook`, when set,
        # is called before every pass that has work (a decode step, a prompt chunk) and is where the ranks agree
        # that a round runs (ep.RoundGate); a rank without work answers with `idle_pass`.
        self.round_hook = None
        if self.ep_state is not None and self.use_graphs and self.scratch_block is not None:
            # The exchange has one shape, so there is one graph; it is built here, where every rank is (its
            # warm-up runs are real exchanges and must happen on all ranks together), with padding rows only.
            self._build_graph(self.max_batch, pad_from=0)
        # per layer: qkv GEMM with norm/RoPE/page write (two kernels for head sizes other than 128), attention +
        # split reduce, o GEMM, norm + router + top-k (one
        # kernel; three where its shape limits do not hold), rank, scatter+quant, expert GEMM x2, combine+norm;
        # + the first norm, lm_head with arg-max and its fold
        self.kernel_launches_per_step = cfg.layers * ((11 if self._fused_router else 13) - (1 if self._fused_qkv else 0)) + 3
        if self.ep_world > 1:
            # the local re-sort of received rows (rank + scatter + row gather), and with the peer-memory
            # transport the two flag exchanges
            self.kernel_launches_per_step += cfg.layers * (3 + (2 if ep_transport == "p2p" else 0))

    # ------------------------------------------------------------------ step
    def _forward(self, tokens, pos, table, attn_ws, moe_ws, split_tokens, ep: bool, pairs: bool = False,
                 chunk_of: tuple[int, int] | None = None, decode_attn: tuple[int, torch.Tensor] | None = None
                 ) -> torch.Tensor:
        """The layer stack for R rows: row i is token `tokens[i]` at position `pos[i]` of the sequence whose
        pages are `table[i]`; it attends to positions 0..pos[i].  Decode passes one row per sequence; a prompt
        chunk passes one row per prompt token with the sequence's table repeated - the same kernels, reading
        the pages in place either way.  `chunk_of` = (first position, rows): the first `rows` rows are
        consecutive prompt tokens of ONE sequence starting there, and attention runs as the tiled causal kernel
        (a page fetched once per 128 score rows) instead of one row per token.  The rows after the chunk are
        padding (expert parallelism) unless `decode_attn` = (split_tokens, workspace) is given: then they are
        decode rows of other sequences, each with its own table row and position, and the decode kernel runs for
        them beside the chunk's (a mixed pass).
        Returns the final normed hidden states [R, hidden].

        Per layer: qkv GEMM, fused q/k norm + RoPE + page write, paged attention, o GEMM, fused
        residual+RMSNorm, router GEMM, FP8 MoE whose combine adds into the residual stream `x`
        (in place) and applies the next layer's input norm."""
        cfg = self.cfg
        D, Hq, Hkv = cfg.head_dim, cfg.q_heads, cfg.kv_heads
        R = tokens.shape[0]
        new_len = pos + 1
        x = self.embed[tokens]
        h = ops.add_rmsnorm(x, None, self.layers[0].ln1, cfg.rms_eps)
        for li, w in enumerate(self.layers):
            if self._fused_qkv:
                # projection with q/k norm, RoPE and the K/V page write in its epilogue
                q = ops.qkv_rope_append_gemm(h, w.wqkv, w.q_norm, w.k_norm, self.cos, self.sin, pos, table,
                                             self.k_pools[li], self.v_pools[li], Hq, cfg.rms_eps, self.gemm_status)
            else:
                qkv = ops.dense_gemm(h, w.wqkv, status=self.gemm_status, workspace=self.gemm_ws).view(R, Hq + 2 * Hkv, D)
                q = ops.qk_norm_rope_append(qkv, w.q_norm, w.k_norm, self.cos, self.sin, pos, table, self.k_pools[li],
                                            self.v_pools[li], Hq, cfg.rms_eps, attn_ws)
            if chunk_of is not None:
                first_pos, n_real = chunk_of
                attn = q.new_zeros(R, Hq, D) if n_real < R and decode_attn is None else torch.empty_like(q)
                ops.paged_attn_prefill(q[:n_real], self.k_pools[li], self.v_pools[li], table[0], first_pos, self.scale,
                                       attn_ws, out=attn[:n_real])
                if decode_attn is not None and n_real < R:
                    ops.paged_attn_decode(q[n_real:], self.k_pools[li], self.v_pools[li], table[n_real:],
                                          new_len[n_real:], self.scale, decode_attn[0], decode_attn[1],
                                          out=attn[n_real:])
            else:
                attn = ops.paged_attn_decode(q, self.k_pools[li], self.v_pools[li], table, new_len, self.scale,
                                             split_tokens, attn_ws, pairs=pairs)
            o = ops.dense_gemm(attn.view(R, Hq * D), w.wo, status=self.gemm_status, workspace=self.gemm_ws)
            nxt = self.layers[li + 1].ln1 if li + 1 < len(self.layers) else self.final_norm
            if self._fused_router:
                # residual add + norm + router projection + top-k in one kernel; the logits stay on the chip (fp32)
                h2, ids, wts = ops.add_rmsnorm_route(x, o, w.ln2, cfg.rms_eps, w.router, cfg.top_k, cfg.norm_topk_prob,
                                                     self.n_valid if ep else None)
                logits, routing = None, (ids, wts)
            else:
                h2 = ops.add_rmsnorm(x, o, w.ln2, cfg.rms_eps)
                logits = ops.dense_gemm(h2, w.router, status=self.gemm_status, workspace=self.gemm_ws)  # bf16, routed as is
                routing = None
            # MoE layer; its combine also adds into the residual stream and applies the next norm
            if ep:
                h = self._ep_moe(h2, logits, w, x, nxt, R, routing)  # rows >= n_valid take no part
            elif routing is not None:
                h = ops.moe_fp8_forward(h2, None, w.w13, w.w13_scale, w.w2, w.w2_scale, cfg.top_k, cfg.norm_topk_prob,
                                        moe_ws, residual=x, norm_weight=nxt, eps=cfg.rms_eps, routing=routing)
            else:
                h = ops.moe_fp8_forward(h2, logits, w.w13, w.w13_scale, w.w2, w.w2_scale, cfg.top_k,
                                        cfg.norm_topk_prob, moe_ws, residual=x, norm_weight=nxt, eps=cfg.rms_eps)
        return h

    def _attn_for(self, rows: int) -> tuple[int, torch.Tensor]:
        """(split_tokens, workspace) of the attention kernel for a step of `rows` rows."""
        pair = self._attn_by_rows.get(rows)
        if pair is None:
            cfg = self.cfg
            split = self._fixed_split or ops.default_split_tokens(rows, cfg.kv_heads, self.max_pages * PAGE)
            pair = (split, ops.paged_attn_workspace(rows, cfg.q_heads, cfg.head_dim, self.max_pages, PAGE, split,
                                                    self.device))
            self._attn_by_rows[rows] = pair
        return pair

    def check_status(self, where: str = "decode engine") -> None:
        """Synchronise and raise if any kernel of this engine has recorded a device-side finding: a block id,
        length or expert id outside its range (the kernels clamp or skip those, so the tokens are wrong), a
        bounded wait that ran out, or an expert-parallel dispatch that overflowed its capacity (the dropped
        pairs contribute nothing)."""
        for rows, (_, ws) in self._attn_by_rows.items():
            ops.read_status(ws, f"{where}: attention ({rows} rows)")
        ops.read_status(self.moe_ws, f"{where}: MoE")
        ops.read_status(self.gemm_status, f"{where}: dense projections")
        for name, what in (("_prefill_attn_ws", "prompt pass (attention)"), ("_prefill_moe_ws", "prompt pass (MoE)"),
                           ("_mixed_attn_ws", "mixed pass (prompt attention)"), ("_mixed_moe_ws", "mixed pass (MoE)")):
            ws = getattr(self, name, None)
            if ws is not None:
                ops.read_status(ws, f"{where}: {what}")
        st = self.ep_state
        if st is not None:
            if getattr(st, "arena", None) is not None:
                ops.read_status(st.status, f"{where}: peer-memory exchange")
            for name in ("perm_send", "perm_local"):
                perm = getattr(st, name, None)
                if perm is not None:
                    ops.read_status(perm.workspace, f"{where}: expert-parallel {name}")
            if bool(st.overflow.item()):
                raise RuntimeError(f"{where}: expert-parallel dispatch overflowed its per-destination capacity of "
                                   f"{st.C} rows; the dropped (token, expert) pairs were left out of the result. "
                                   "Build the engine with a larger ep_capacity.")

    def copy_kv_tokens(self, src: list[tuple[int, int]], dst: list[tuple[int, int]]) -> None:
        """Copy the K/V of single tokens between page slots, in every layer: src[i] = (block, slot) ->
        dst[i].  Used when a prefix-cache hit ends in, or runs through, a partially filled block: those tokens
        are compacted into the row's own pages instead of being recomputed."""
        if len(src) != len(dst):
            raise ValueError("src and dst must list the same number of tokens")
        if not src:
            return
        dev = self.k_pools[0].device
        sb = torch.tensor([b for b, _ in src], device=dev)
        ss = torch.tensor([s for _, s in src], device=dev)
        db = torch.tensor([b for b, _ in dst], device=dev)
        ds = torch.tensor([s for _, s in dst], device=dev)
        for kp, vp in zip(self.k_pools, self.v_pools):
            kp[db, :, ds, :] = kp[sb, :, ss, :]
            vp[db, :, ds, :] = vp[sb, :, ss, :]

    def _step_eager(self, B: int) -> None:
        """One decode step over rows [0, B) of the static buffers; advances ctx_lens by one."""
        split, attn_ws = self._attn_for(B)
        h = self._forward(self.tokens[:B], self.ctx_lens[:B], self.block_table[:B], attn_ws, self.moe_ws,
                          split, self.ep_state is not None)
        if self.keep_logits:
            self.last_logits = ops.dense_gemm(h, self.lm_head, status=self.gemm_status)
        ops.lm_head_argmax(h, self.lm_head, self.argmax_ws, out=self.next_tokens[:B], status=self.gemm_status)
        self.ctx_lens[:B] += 1

    def _ep_moe(self, h2, logits, w: LayerWeights, x, next_norm, B: int, routing=None) -> torch.Tensor:
        """Expert-parallel MoE layer: dispatch and combine around the local grouped GEMMs, by NCCL all-to-all
        or, with a peer arena, by stores into the other ranks' memory.  The exchange has one fixed shape (the
        engine's full batch on every rank); a pass with fewer real rows runs it with padding rows that the
        router leaves without an expert (`n_valid`)."""
        import torch.distributed as dist

        from . import ep
        st = self.ep_state
        if B != st.T:
            raise ValueError("an expert-parallel pass runs at the exchange's full shape; pad it (see step / prefill)")
        return ep.ep_moe_forward(st, h2, logits, w.w13, w.w13_scale, w.w2, w.w2_scale, self.cfg.norm_topk_prob, ops,
                                 lambda o, i: dist.all_to_all_single(o, i, group=st.group), residual=x,
                                 norm_weight=next_norm, eps=self.cfg.rms_eps, n_valid=self.n_valid, routing=routing)

    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024)

    def graph_batch(self, B: int) -> int:
        """Rows the captured graph for a batch of B runs: B itself, or with a scratch page the next bucket, so
        that a batch whose size changes with every admitted and finished request reuses a handful of graphs."""
        if self.ep_state is not None:
            if self.scratch_block is None and B != self.max_batch:
                raise ValueError("this expert-parallel engine reads pools it does not own (no scratch page for "
                                 "padding rows), so it can only step at its full batch")
            return self.max_batch  # the exchange has one shape; fewer rows are padded up to it
        if self.scratch_block is None:
            return B
        for b in self.GRAPH_BUCKETS:
            if b >= B:
                return min(b, self.max_batch)
        return self.max_batch

    def _pad_rows(self, lo: int, hi: int) -> None:
        """Make rows [lo, hi) of the static state padding rows: token 0 at position 0 of a sequence whose only
        page is the scratch page."""
        if hi > lo:
            self.tokens[lo:hi] = 0
            self.ctx_lens[lo:hi] = 0
            self.block_table[lo:hi, 0] = self.scratch_block

    def _build_graph(self, B: int, pad_from: int | None = None) -> torch.cuda.CUDAGraph:
        """Capture the step for B rows (two eager warm-up runs, then the capture).  `pad_from`: rows from
        there on are set up as padding rows first."""
        if pad_from is not None:
            self._pad_rows(pad_from, B)
            self.n_valid.fill_(pad_from)
        saved = self.ctx_lens.clone()
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up: library handles, function attributes, tensor maps
                self._step_eager(B)
                # every warm-up run writes the K/V slot of the CURRENT position only (the one the real step
                # will overwrite): a run that advanced could cross into a page the row does not own yet
                self.ctx_lens.copy_(saved)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step_eager(B)
        self.ctx_lens.copy_(saved)  # warm-up and capture advanced nothing the caller asked for
        torch.cuda.synchronize()
        self._graphs[B] = g
        return g

    def step(self, B: int, joined: bool = False) -> torch.Tensor:
        """Run one decode step for the first B rows of the static state; returns next tokens (device).
        On an expert-parallel engine B may be anything from 0 (an idle rank keeping the exchange company) to
        the full batch; `joined` says the caller has already agreed the round with the other ranks."""
        lowest = 0 if self.ep_state is not None else 1
        if B < lowest or B > self.max_batch:
            raise ValueError(f"batch {B} outside [{lowest}, {self.max_batch}]")
        if not self.use_graphs and self.ep_state is None:
            self._step_eager(B)
            return self.next_tokens[:B]
        rows = self.graph_batch(B)
        if self.ep_state is not None:
            if self.round_hook is not None and not joined:
                self.round_hook()
            self.n_valid.fill_(B)
        if rows > B:
            # padding rows: reset every step because the graph advances their lengths like everyone's
            self._pad_rows(B, rows)
        real, B = B, rows
        if not self.use_graphs:
            self._step_eager(B)
            return self.next_tokens[:real]
        g = self._graphs.get(B)
        if g is None:
            g = self._build_graph(B)
        g.replay()
        return self.next_tokens[:real]

    def idle_pass(self) -> None:
        """Expert parallelism: take part in one exchange round without any rows of one's own."""
        self.step(0, joined=True)

    # --------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill(self, token_ids: list[int], block_ids: list[int], cached_tokens: int = 0,
                chunk: int = 1024) -> tuple[int, torch.Tensor]:
        """Prompt pass for one sequence; writes K/V of tokens [cached_tokens, n) into `block_ids` pages.

        Runs in chunks of `chunk` prompt tokens through the same projection, glue and MoE kernels as decode
        (every token of a chunk is a row with its own position); attention reads the sequence's pages in place,
        cached prefix pages included - there is no dense gather of the KV as in the reference
        (src/inference_server/kv_cache/hf_format.py:21-45).  The K/V of a whole chunk are written to their page
        slots before the chunk's attention runs.  Attention is the tiled causal kernel
        (b200_paged_attn_prefill: a page fetched once per 128 score rows); for head shapes it is not built for,
        the decode kernel with one row per token (two rows per CTA: b200_paged_attn_decode_pairs), where
        row i only looks at positions <= its own, which is the causal mask.
        Under expert parallelism a chunk is one exchange round like a decode step: it is padded to the
        exchange's fixed shape (the engine's full batch) with rows that route nowhere, and the other ranks spend
        the round on a decode step, a chunk of their own or an idle pass.
        Returns (first generated token, last-position logits - None unless the engine was built with keep_logits)."""
        n = len(token_ids)
        if n == 0 or cached_tokens >= n:
            raise ValueError("prefill needs at least one uncached token")
        if len(block_ids) * PAGE < n:
            raise ValueError("not enough pages for the prompt")
        if len(block_ids) > self.max_pages:
            raise ValueError("sequence needs more pages than the block table is wide")
        ep = self.ep_state is not None
        if ep:
            if self.scratch_block is None:
                raise ValueError("prompt passes on an expert-parallel engine need the engine's own pools (a scratch "
                                 "page for the padding rows)")
            chunk = self.ep_state.T
        cfg = self.cfg
        tiled = ops.paged_attn_prefill_supported(cfg.q_heads, cfg.kv_heads, cfg.head_dim, PAGE, torch.bfloat16)
        if getattr(self, "_prefill_chunk", 0) != chunk:
            self._prefill_chunk = chunk
            self._prefill_split = ops.default_split_tokens(chunk, cfg.kv_heads, self.max_pages * PAGE)
            # the tiled kernel needs no workspace beyond a status word; the row-per-token form needs the split
            # partials of `chunk` rows
            self._prefill_attn_ws = torch.zeros(256, dtype=torch.uint8, device=self.device) if tiled else \
                ops.paged_attn_workspace(chunk, cfg.q_heads, cfg.head_dim, self.max_pages, PAGE, self._prefill_split,
                                         self.device)
            self._prefill_moe_ws = None if ep else ops.moe_fp8_workspace(chunk, cfg.experts, cfg.top_k, cfg.hidden,
                                                                         cfg.moe_inter, self.device)
        # consecutive prompt tokens share the table, so the row-per-token form takes them two rows per CTA where it can
        pairs = not tiled and ops.paged_attn_pairs_supported(cfg.q_heads, cfg.kv_heads, cfg.head_dim, PAGE, torch.bfloat16)
        row = torch.zeros(self.max_pages, dtype=torch.int32)
        row[: len(block_ids)] = torch.tensor(block_ids, dtype=torch.int32)
        row = row.to(self.device)
        h_last = None
        for lo in range(cached_tokens, n, chunk):
            hi = min(n, lo + chunk)
            tokens = torch.tensor(token_ids[lo:hi], device=self.device)
            pos = torch.arange(lo, hi, device=self.device, dtype=torch.int32)
            table = row.unsqueeze(0).expand(hi - lo, -1).contiguous()
            if ep:
                pad = chunk - (hi - lo)
                if pad:
                    tokens = torch.cat([tokens, tokens.new_zeros(pad)])
                    pos = torch.cat([pos, pos.new_zeros(pad)])
                    scratch = torch.zeros(pad, self.max_pages, dtype=torch.int32, device=self.device)
                    scratch[:, 0] = self.scratch_block
                    table = torch.cat([table, scratch])
                if self.round_hook is not None:
                    self.round_hook()
                self.n_valid.fill_(hi - lo)
            h = self._forward(tokens, pos, table, self._prefill_attn_ws, self._prefill_moe_ws, self._prefill_split,
                              ep, pairs=pairs, chunk_of=(lo, hi - lo) if tiled else None)
            h_last = h[hi - lo - 1:hi - lo].contiguous()
        first = ops.lm_head_argmax(h_last, self.lm_head, self.argmax_ws, status=self.gemm_status)
        # the logits cost a second pass over lm_head: only for engines built to keep them (tests, debugging)
        logits = ops.dense_gemm(h_last, self.lm_head, status=self.gemm_status)[0] if self.keep_logits else None
        return int(first[0]), logits

    @torch.no_grad()
    def mixed_step(self, B: int, chunk_token_ids: list[int], block_ids: list[int], first_pos: int,
                   want_first: bool = True) -> tuple[torch.Tensor, int | None, torch.Tensor | None]:
        """One pass that is a decode step for rows [0, B) of the static state AND a prompt chunk of one other
        sequence: its tokens `chunk_token_ids` sit at positions first_pos.. of the sequence whose pages are
        `block_ids` (earlier positions already written).  The reference runs the two as separate forwards
        (src/inference_server/scheduler.py:312-353 then :379-402) and names the merged form as the next step
        (docs/arch-scheduler.html:269-270); merged, the projections' and the experts' weights are streamed once
        for both, which is most of what a decode step costs.  The chunk's rows come first; every kernel but
        attention treats the rows alike, and attention runs as the tiled causal kernel for the chunk and the
        decode kernel for the rest.
        Returns (next tokens of the B decode rows (device), token after the chunk's last position, its logits);
        the last two are None unless `want_first` (the logits also unless the engine was built with keep_logits).
        Advances ctx_lens of the decode rows by one."""
        n = len(chunk_token_ids)
        if self.ep_state is not None:
            raise ValueError("mixed passes are not built for expert-parallel engines: run the chunk and the step as "
                             "two rounds")
        if n == 0 or B < 1 or B > self.max_batch:
            raise ValueError(f"mixed pass needs a chunk and 1..{self.max_batch} decode rows (got {n} and {B})")
        if len(block_ids) * PAGE < first_pos + n or len(block_ids) > self.max_pages:
            raise ValueError("the chunk's sequence needs more pages than it was given or than the block table is wide")
        cfg = self.cfg
        if not ops.paged_attn_prefill_supported(cfg.q_heads, cfg.kv_heads, cfg.head_dim, PAGE, torch.bfloat16):
            raise ValueError("mixed passes need the tiled prompt-attention kernel, which is not built for this head shape")
        R = n + B
        if getattr(self, "_mixed_rows", 0) < R:
            self._mixed_rows = max(R, 2 * getattr(self, "_mixed_rows", 0))
            self._mixed_moe_ws = ops.moe_fp8_workspace(self._mixed_rows, cfg.experts, cfg.top_k, cfg.hidden,
                                                       cfg.moe_inter, self.device)
            self._mixed_attn_ws = torch.zeros(256, dtype=torch.uint8, device=self.device)  # status word only
        row = torch.zeros(self.max_pages, dtype=torch.int32)
        row[: len(block_ids)] = torch.tensor(block_ids, dtype=torch.int32)
        row = row.to(self.device)
        tokens = torch.cat([torch.tensor(chunk_token_ids, device=self.device), self.tokens[:B]])
        pos = torch.cat([torch.arange(first_pos, first_pos + n, device=self.device, dtype=torch.int32), self.ctx_lens[:B]])
        table = torch.cat([row.unsqueeze(0).expand(n, -1), self.block_table[:B]])
        h = self._forward(tokens, pos, table, self._mixed_attn_ws, self._mixed_moe_ws, 0, False, chunk_of=(first_pos, n),
                          decode_attn=self._attn_for(B))
        first = logits = None
        if want_first:
            # the chunk's last row and the decode rows are neighbours: lm_head is streamed once for both
            nxt = ops.lm_head_argmax(h[n - 1:], self.lm_head, self.argmax_ws, status=self.gemm_status)
            self.next_tokens[:B].copy_(nxt[1:])
            first = int(nxt[0])
        else:
            ops.lm_head_argmax(h[n:], self.lm_head, self.argmax_ws, out=self.next_tokens[:B], status=self.gemm_status)
        if want_first and self.keep_logits:
            logits = ops.dense_gemm(h[n - 1:n], self.lm_head, status=self.gemm_status)[0]
        self.ctx_lens[:B] += 1
        return self.next_tokens[:B], first, logits

    # ------------------------------------------------------------- accounting
    def weight_bytes_per_step(self, experts_hit_per_layer: float | None = None) -> dict:
        """Bytes one decode step must stream from HBM, by stream (for the step roofline)."""
        cfg = self.cfg
        per_expert = 3 * cfg.hidden * cfg.moe_inter
        hit = cfg.experts if experts_hit_per_layer is None else experts_hit_per_layer
        dense = ((cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim * cfg.hidden + cfg.hidden * cfg.q_heads * cfg.head_dim
                 + cfg.experts * cfg.hidden) * 2
        return {
            "experts": cfg.layers * hit * per_expert,
            "dense": cfg.layers * dense,
            "lm_head": cfg.vocab_size * cfg.hidden * 2,
            "kv_per_token": cfg.layers * 2 * cfg.kv_heads * cfg.head_dim * 2,
        }


def kv_bytes_per_token_layer(cfg: ModelConfig) -> int:
    return 2 * cfg.kv_heads * cfg.head_dim * 2


def pages_for(tokens: int) -> int:
    return math.ceil(tokens / PAGE)

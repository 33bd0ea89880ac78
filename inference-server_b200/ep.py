"""Expert-parallel dispatch planning (host/torch index arithmetic, no kernels).

Experts are partitioned by id: rank r of W owns experts [r*E/W, (r+1)*E/W).  Each
rank routes its own tokens, sorts the (token, slot) pairs by expert id (which is
also by destination rank) and exchanges rows with fixed-capacity all-to-alls so
that no step needs a host round trip:

    send buffer  [W, capacity, hidden]   slot s of segment d = the s-th pair of
                                         this rank that goes to rank d
    slot_of_pair [T*K]                   d * capacity + s for every pair
    expert_of_slot [W*capacity]          local expert id at the destination, or
                                         E_local for an empty slot

On the GPU the slot placement is done inside the scatter+quantise kernel
(``b200_moe_permute_quant_ep``); ``plan_dispatch`` is the same arithmetic in torch
ops, used by the CPU stand-in kernels of the gloo tests and as a cross-check.

Two transports move the rows.  "a2a": local send buffers and a library all-to-all
(NCCL on GPUs, gloo in the CPU tests).  "p2p": every rank keeps its receive buffers in
one allocation that the other ranks of the node map (``PeerArena``), the dispatch
kernel and the down-GEMM epilogue store rows straight into the owner's memory over
NVLink, and a flag exchange (``ep_barrier``) orders those stores before the reads - no
library collective and no staging copy on the data path.
"""
from __future__ import annotations

import torch


def default_capacity(num_tokens: int, top_k: int, world: int, factor: float = 2.0) -> int:
    """Rows reserved per (source, destination) pair: `factor` x the mean, rounded up to 16."""
    mean = num_tokens * top_k / world
    cap = int(mean * factor + 15) // 16 * 16
    return max(16, min(cap, num_tokens * top_k))


def plan_dispatch(topk_ids: torch.Tensor, row_of_pair: torch.Tensor, expert_offsets: torch.Tensor,
                  num_experts: int, world: int, capacity: int):
    """Index arrays for the fixed-capacity exchange.

    topk_ids [T, K] int32 (global expert ids), row_of_pair [T*K] int32 (position in the
    expert-sorted order), expert_offsets [E+1] int32.
    Returns (slot_of_pair [T*K] int64, expert_of_slot [W*capacity] int32, overflow scalar bool tensor).
    Pairs beyond `capacity` for a destination are dropped into slot -1 and flagged; pairs with expert id -1
    (padding rows) get slot -1 without a flag."""
    e_local = num_experts // world
    flat = topk_ids.reshape(-1).long()
    real = flat >= 0  # id -1 is "no expert" (a padding row): the pair is neither sent nor counted
    safe = torch.where(real, flat, torch.zeros_like(flat))
    dst = safe // e_local
    seg_start = expert_offsets.long()[dst * e_local]
    pos = row_of_pair.long() - seg_start
    fits = real & (pos < capacity)
    overflow = (real & ~fits).any()
    flat = safe
    slot = torch.where(fits, dst * capacity + pos, torch.full_like(pos, -1))
    # fixed shapes only (the step is captured in a CUDA graph): overflowed pairs write to a spare last entry
    trash = world * capacity
    expert_of_slot = torch.full((trash + 1,), e_local, dtype=torch.int32, device=topk_ids.device)
    expert_of_slot.index_copy_(0, torch.where(fits, slot, torch.full_like(slot, trash)), (flat % e_local).to(torch.int32))
    expert_of_slot[trash:].fill_(e_local)  # (a fill kernel: a scalar assignment would be a host copy)
    return slot, expert_of_slot[:trash], overflow


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerArena:
    """One device allocation per rank holding the receive side of the peer-memory exchange, with the same
    layout on every rank, plus the addresses of the other ranks' arenas as mapped into this process.

    Layout (each section 256-byte aligned): xq_recv [W*C, H] u8 | xs_recv [W*C, H/128] f32 | id_recv [W*C] i32 |
    y_recv [W*C, H] bf16 | flags [2 phases][8] i32."""

    def __init__(self, hidden: int, world: int, capacity: int, device):
        rows = world * capacity
        self.rows, self.hidden, self.world = rows, hidden, world
        self.off_xq = 0
        self.off_xs = _align(self.off_xq + rows * hidden)
        self.off_id = _align(self.off_xs + rows * (hidden // 128) * 4)
        self.off_y = _align(self.off_id + rows * 4)
        self.off_flags = _align(self.off_y + rows * hidden * 2)
        self.nbytes = self.off_flags + 256
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        self.rank = 0
        self.bases = [self.buf.data_ptr()]  # arena address of every rank, as seen from this process
        self._opened: list[int] = []
        self.failures: list[str] = []

    def view(self, off: int, nbytes: int, dtype, shape):
        return self.buf[off:off + nbytes].view(dtype).view(shape)

    def connect(self, ops, group) -> bool:
        """Exchange CUDA IPC handles over `group` and map every other rank's arena (ranks of one node).
        Collective.  Returns True when EVERY rank mapped every peer; if any rank could not export or map
        (no peer access, IPC closed in this container), all ranks unmap what they have and return False
        together, so the caller can fall back to the all-to-all transport on every rank alike."""
        import torch.distributed as dist

        world = dist.get_world_size(group)
        if world != self.world:
            raise ValueError(f"arena laid out for {self.world} ranks, group has {world}")
        self.rank = dist.get_rank(group)
        try:
            mine = ops.ipc_export(self.buf)
        except Exception as exc:  # reported below, after every rank has joined the exchange
            mine = ("error", repr(exc))
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        ok = all(e[0] != "error" for e in everyone)
        self.bases = []
        if ok:
            try:
                for r, (handle, offset) in enumerate(everyone):
                    if r == self.rank:
                        self.bases.append(self.buf.data_ptr())
                    else:
                        base, ptr = ops.ipc_import(handle, offset)
                        self._opened.append(base)
                        self.bases.append(ptr)
            except Exception as exc:
                ok = False
                mine = ("error", repr(exc))
        verdicts = [None] * world
        dist.all_gather_object(verdicts, mine if not ok else ("ok", ""), group=group)
        self.failures = [f"rank {r}: {v[1]}" for r, v in enumerate(verdicts) if v[0] == "error"]
        if self.failures:
            self.close(ops)
            self.bases = [self.buf.data_ptr()]
            return False
        dist.barrier(group=group)  # nobody proceeds (or frees) before every mapping exists
        return True

    def connect_in_process(self, arenas: list["PeerArena"], rank: int) -> None:
        """Several ranks emulated in one process (tests on one GPU): peers are plain device pointers."""
        self.rank = rank
        self.bases = [a.buf.data_ptr() for a in arenas]

    def close(self, ops) -> None:
        for base in self._opened:
            ops.ipc_close(base)
        self._opened = []


class EPState:
    """Per-rank buffers of the expert-parallel exchange, allocated once (graph-capturable).
    With `arena` (a connected PeerArena) the exchange runs over peer memory, else over `all_to_all`."""

    def __init__(self, num_tokens: int, hidden: int, top_k: int, num_experts: int, world: int, capacity: int,
                 device, group=None, arena: PeerArena | None = None):
        self.T, self.H, self.K, self.E, self.W, self.C = num_tokens, hidden, top_k, num_experts, world, capacity
        self.e_local = num_experts // world
        self.group = group
        self.arena = arena
        rows = world * capacity
        u8, f32, i32 = torch.uint8, torch.float32, torch.int32
        self.overflow = torch.zeros(1, dtype=i32, device=device)  # sticky: set when a destination's capacity ran out
        # permutation buffers, allocated once when the kernels are the real ones (a hot path must not allocate
        # or clear anything per layer); None lets a stand-in allocate per call
        self.perm_send = self.perm_local = self.slot_of_pair = None
        if torch.device(device).type == "cuda":
            from . import ops
            self.perm_send = ops.new_permutation(num_tokens, top_k, num_experts, device)
            self.perm_local = ops.new_permutation(rows, 1, self.e_local + 1, device)
            self.slot_of_pair = torch.empty(num_tokens * top_k, dtype=i32, device=device)
        self.xq_sorted = torch.zeros(rows, hidden, dtype=u8, device=device)
        self.xs_sorted = torch.zeros(rows, hidden // 128, dtype=f32, device=device)
        if arena is not None:
            if arena.rows != rows or arena.hidden != hidden:
                raise ValueError("arena was laid out for other sizes")
            a = arena
            self.rank = a.rank
            self.xq_recv = a.view(a.off_xq, rows * hidden, u8, (rows, hidden))
            self.xs_recv = a.view(a.off_xs, rows * (hidden // 128) * 4, f32, (rows, hidden // 128))
            self.id_recv = a.view(a.off_id, rows * 4, i32, (rows,))
            self.y_recv = a.view(a.off_y, rows * hidden * 2, torch.bfloat16, (rows, hidden))
            self.flags = [a.view(a.off_flags + 32 * ph, 32, i32, (8,)) for ph in range(2)]
            self.peer_xq = [b + a.off_xq for b in a.bases]
            self.peer_xs = [b + a.off_xs for b in a.bases]
            self.peer_id = [b + a.off_id for b in a.bases]
            self.peer_y = [b + a.off_y for b in a.bases]
            self.peer_flags = [[b + a.off_flags + 32 * ph for b in a.bases] for ph in range(2)]
            self.epochs = torch.zeros(2, dtype=i32, device=device)  # local: exchanges done so far, per phase
            self.status = torch.zeros(64, dtype=i32, device=device)
            return
        self.xq_send = torch.zeros(rows, hidden, dtype=u8, device=device)
        self.xq_recv = torch.zeros(rows, hidden, dtype=u8, device=device)
        self.xs_send = torch.zeros(rows, hidden // 128, dtype=f32, device=device)
        self.xs_recv = torch.zeros(rows, hidden // 128, dtype=f32, device=device)
        self.id_send = torch.zeros(rows, dtype=i32, device=device)
        self.id_recv = torch.zeros(rows, dtype=i32, device=device)
        self.y_send = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=device)
        self.y_recv = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=device)


def ep_moe_forward(st: EPState, h, logits, w13, w13_scale, w2, w2_scale, renormalize, kernels, all_to_all,
                   residual=None, norm_weight=None, eps: float = 1e-6, n_valid=None, routing=None):
    """One expert-parallel FP8 MoE layer on this rank's tokens `h` [T, H].

    `w13/w2` hold only this rank's experts.  `kernels` supplies the compute steps (the ``ops`` module on a
    GPU; a CPU stand-in in the gloo tests) and `all_to_all(out, inp)` the equal-split exchange.  Steps:
      1. route; sort by (global) expert id, quantise and place every row in its fixed-capacity send slot
         (one kernel: the sort by expert is also a sort by owner rank);
      2. all-to-all of e4m3 rows, scales and owner-local expert ids (empty slots carry the id E_local);
      3. stable sort of the received slots by local expert fused with the row copy into that order (the dummy
         expert E_local sorts last, gets no tiles and is not copied), grouped gate/up GEMM, down GEMM writing
         straight back into slot order;
      4. all-to-all back and weighted combine in the original (token, slot) order.
    Everything has fixed shapes and no host round trip, so the layer can sit inside a captured CUDA graph.
    With a peer arena (`st.arena`) steps 2 and 4 are stores into the other ranks' memory from inside the
    dispatch kernel and the down GEMM, separated by flag exchanges; `all_to_all` is then unused.
    The shapes are the same on every rank and in every pass.  `n_valid` (an int32 scalar on the device) says how
    many leading rows of `h` are real in this pass: the router gives the others no expert, so they are neither
    sent nor combined - a rank with a short batch, or none, still takes part in the exchange.
    `routing` = (ids, weights) when the tokens are routed already (the fused norm + router kernel, which has
    applied `n_valid` itself); `logits` is then unused."""
    if st.arena is not None:
        wts, slot_of_pair = p2p_dispatch(st, h, logits, renormalize, kernels, n_valid, routing)
        kernels.ep_barrier(st.peer_flags[0], st.epochs[0:1], st.rank, st.W, st.status)
        p2p_experts(st, w13, w13_scale, w2, w2_scale, kernels)
        kernels.ep_barrier(st.peer_flags[1], st.epochs[1:2], st.rank, st.W, st.status)
        return _combine(st, wts, slot_of_pair, kernels, residual, norm_weight, eps)
    T, K, W, C, El = st.T, st.K, st.W, st.C, st.e_local
    ids, wts = routing if routing is not None else kernels.moe_route(logits, K, renormalize, n_valid)
    _, slot_of_pair = kernels.moe_permute_quant_ep(ids, h, st.E, W, C, st.xq_send, st.xs_send, st.id_send, st.overflow,
                                                   perm=st.perm_send, slot_of_pair=st.slot_of_pair)
    all_to_all(st.xq_recv, st.xq_send)
    all_to_all(st.xs_recv, st.xs_send)
    all_to_all(st.id_recv, st.id_send)

    lperm = kernels.moe_permute_gather_fp8(st.id_recv, El + 1, El, st.xq_recv, st.xs_recv, st.xq_sorted, st.xs_sorted,
                                           perm=st.perm_local)
    hq, hs = kernels.moe_fp8_gemm_gate_up(st.xq_sorted, st.xs_sorted, w13, w13_scale, lperm)
    kernels.moe_fp8_gemm_down(hq, hs, w2, w2_scale, lperm, out=st.y_send, out_row_map=lperm.sorted_pair_ids)
    all_to_all(st.y_recv, st.y_send)
    return _combine(st, wts, slot_of_pair, kernels, residual, norm_weight, eps)


def _combine(st: EPState, wts, slot_of_pair, kernels, residual, norm_weight, eps):
    """Weighted sum of the returned expert rows in (token, slot) order; pairs that overflowed (slot -1,
    flagged) contribute nothing (the combine kernels skip negative rows)."""
    if residual is not None:
        return kernels.moe_combine_add_rmsnorm(st.y_recv, slot_of_pair, wts, residual, norm_weight, eps)
    return kernels.moe_combine(st.y_recv, slot_of_pair, wts)


# ------------------------------------------------------------ peer-memory transport --
# The three stages of one layer.  Between them stands a flag exchange: ep_barrier in production (every rank
# is its own process and GPU); the single-GPU tests emulate several ranks in one process and therefore run
# stage by stage over all ranks with ep_signal / ep_wait apart (kernels that wait for each other must not
# sit in one stream).

def p2p_dispatch(st: EPState, h, logits, renormalize, kernels, n_valid=None, routing=None):
    """Route (unless `routing` is given), then sort + quantise + store every row, its scales and its expert id
    into the owner's receive buffers (one kernel).  Returns (routing weights, slot_of_pair)."""
    ids, wts = routing if routing is not None else kernels.moe_route(logits, st.K, renormalize, n_valid)
    _, slot_of_pair = kernels.moe_permute_quant_ep_p2p(ids, h, st.E, st.W, st.C, st.rank, st.peer_xq, st.peer_xs,
                                                       st.peer_id, st.overflow, perm=st.perm_send,
                                                       slot_of_pair=st.slot_of_pair)
    return wts, slot_of_pair


def p2p_experts(st: EPState, w13, w13_scale, w2, w2_scale, kernels) -> None:
    """Local experts on the received rows; the down GEMM's epilogue stores each result row into y_recv of the
    rank the row came from."""
    El = st.e_local
    lperm = kernels.moe_permute_gather_fp8(st.id_recv, El + 1, El, st.xq_recv, st.xs_recv, st.xq_sorted, st.xs_sorted,
                                           perm=st.perm_local)
    hq, hs = kernels.moe_fp8_gemm_gate_up(st.xq_sorted, st.xs_sorted, w13, w13_scale, lperm)
    kernels.moe_fp8_gemm_down_p2p(hq, hs, w2, w2_scale, lperm, st.peer_y, lperm.sorted_pair_ids, st.W, st.C, st.rank,
                                  st.status)


# --------------------------------------------------------- agreeing on exchange rounds --
class RoundGate:
    """Host-side agreement of the expert-parallel ranks on whether another exchange round runs.

    Every MoE layer of a pass waits for the other ranks' rows, so all ranks must run the same number of
    passes.  Data-parallel serving gives every rank its own requests: at any moment some ranks have a decode
    step or a prompt chunk to run and others have nothing.  Before every pass each rank calls ``join``; the
    answer is the same on all of them: if any rank has work, every rank runs exactly one pass (those without
    work an idle pass with no rows of their own), otherwise none does.  One small all-reduce over a gloo group
    (host memory, so it never queues behind GPU work)."""

    def __init__(self, group=None):
        import torch.distributed as dist

        ranks = dist.get_process_group_ranks(group) if group is not None else None
        self.group = dist.new_group(ranks=ranks, backend="gloo")  # collective over the default group

    def join(self, have_work: bool, leaving: bool = False) -> tuple[bool, bool]:
        """Collective.  Returns (some rank has work, some rank is leaving).  When a rank is leaving nobody runs
        a pass: the exchange cannot complete without it."""
        import torch.distributed as dist

        t = torch.tensor([int(have_work), int(leaving)], dtype=torch.int32)
        dist.all_reduce(t, group=self.group)
        return bool(t[0] > 0), bool(t[1] > 0)


class RoundKeeper:
    """Keeps one rank in step with the exchange rounds of the others.

    ``work_round`` is what a thread with a pass to run calls first (``DecodeEngine.round_hook``); a background
    thread answers the rounds that other ranks start while this one has nothing to do, by running `idle_pass`.
    Both take `lock` (the backend lock that the scheduler holds for its whole tick), so a rank never has two
    threads inside the gate at once, and the order of its joins is the order of its passes."""

    def __init__(self, gate: RoundGate, idle_pass, lock, idle_sleep: float = 0.002):
        import threading

        self.gate, self.idle_pass, self.lock, self.idle_sleep = gate, idle_pass, lock, idle_sleep
        self.rounds = 0       # passes this rank has run, with or without rows of its own
        self.idle_rounds = 0
        self.peer_left = False
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._idle_loop, name="ep-round-keeper", daemon=True)

    def start(self) -> "RoundKeeper":
        self._thread.start()
        return self

    def work_round(self) -> None:
        """Agree a round for a pass of this rank; the caller holds `lock`."""
        if self.peer_left:
            raise RuntimeError("a rank has left the expert-parallel group; no further exchange can complete")
        _, left = self.gate.join(True)
        if left:
            self.peer_left = True
            raise RuntimeError("a rank has left the expert-parallel group; no further exchange can complete")
        self.rounds += 1

    def _idle_loop(self) -> None:
        import time

        while not self._stop.is_set():
            ran = False
            with self.lock:
                if self._stop.is_set() or self.peer_left:
                    break
                work, left = self.gate.join(False)
                if left:
                    self.peer_left = True
                    break
                if work:
                    self.idle_pass()
                    self.rounds += 1
                    self.idle_rounds += 1
                    ran = True
            # out of the lock: give a thread with work the chance to take it
            time.sleep(self.idle_sleep / 10 if ran else self.idle_sleep)

    def close(self) -> None:
        """Tell the other ranks this one is going and stop answering rounds.  Collective in effect: the others
        see `leaving` at their next join, whoever starts it."""
        self._stop.set()
        with self.lock:
            if not self.peer_left:
                self.gate.join(False, leaving=True)
                self.peer_left = True
        if self._thread.is_alive():
            self._thread.join(timeout=5)

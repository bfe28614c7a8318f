"""Expert-parallel load balancing (EPLB): redundant expert replicas, load statistics, periodic re-placement.

With expert parallelism every rank owns ``num_local`` expert slots.  Token routing is skewed - a few experts take a
large share of the pairs - so the rank that owns a hot expert sets the time of every MoE layer.  EPLB adds ``R``
redundant slots: ``P = E + R`` *physical* experts hold the ``E`` *logical* ones, hot experts in several copies, and
the copies are packed onto the ranks so that the expected pairs per rank are even.  The layer keeps routing on logical
ids and spreads the pairs of a replicated expert over its copies.

Pieces:

* :func:`rebalance` - pure function ``load [E] -> phy2log [P]``: replicate by greatest load per copy, pack by
  longest-processing-time onto ranks with a fixed number of slots, then keep experts that stay on a rank in the slot
  they already occupy so that re-placement moves as few weights as possible.
* :func:`build_maps` - ``phy2log -> (log2phy [E, max_copies], logcnt [E])`` used by the layer at routing time.
* :class:`EplbState` - owned by the model runner: sums the per-layer logical load of the last ``window`` steps,
  and every ``step_interval`` steps all-reduces it over the EP group (every rank then computes the same placement),
  rebalances every layer and moves expert weights between ranks (:func:`rearrange_layer`: local copies where the
  expert already lives on the rank, one batched send / receive round otherwise).  Weights move in place, routing maps
  are device buffers updated in place, so captured CUDA graphs stay valid.

All ranks of the EP group call :meth:`EplbState.step` once per engine step (the replicas of a data-parallel
deployment step in lock-step), so the re-placement rounds line up without extra coordination.

Parity: the reference's MoE models implement upstream's ``MixtureOfExperts`` EPLB interface
(vllm_metax/models/deepseek_v2.py:327-337 physical / logical / redundant expert counts, :1745-1772
``set_eplb_state`` / ``update_physical_experts_metadata``; vllm_metax/models/deepseek_v4/model.py has the same
hooks) and rely on upstream's balancer and weight shuffle; this module is both.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist


def initial_placement(num_logical: int, num_physical: int) -> torch.Tensor:
    """``phy2log`` before any statistics exist: every expert once, the redundant slots repeat experts 0, 1, ..."""
    assert num_physical >= num_logical
    extra = torch.arange(num_physical - num_logical, dtype=torch.int64) % num_logical
    return torch.cat([torch.arange(num_logical, dtype=torch.int64), extra])


def replicate(load: torch.Tensor, num_physical: int) -> torch.Tensor:
    """Copies per logical expert (sum = ``num_physical``): each redundant slot goes to the expert whose load per copy
    is greatest.  Ties go to the lower id (deterministic on every rank)."""
    E = load.numel()
    cnt = torch.ones(E, dtype=torch.int64)
    w = load.double().clone()
    for _ in range(num_physical - E):
        e = int(torch.argmax(w / cnt))          # argmax returns the first maximum
        cnt[e] += 1
    return cnt


def rebalance(load: torch.Tensor, num_physical: int, num_ranks: int,
              old_phy2log: Optional[torch.Tensor] = None) -> torch.Tensor:
    """New ``phy2log [P]`` for one layer.  ``load [E]``: pairs routed to each logical expert in the window."""
    E = load.numel()
    assert num_physical % num_ranks == 0 and num_physical >= E
    per = num_physical // num_ranks
    load = load.double().cpu()
    cnt = replicate(load, num_physical)
    # one item per copy, weight = the expert's load shared between its copies
    items = [(float(load[e]) / int(cnt[e]), e) for e in range(E) for _ in range(int(cnt[e]))]
    items.sort(key=lambda it: (-it[0], it[1]))
    rank_load = [0.0] * num_ranks
    rank_items: list[list[int]] = [[] for _ in range(num_ranks)]
    for w, e in items:
        # least-loaded rank with a free slot; a rank that already holds a copy of e is avoided when another is as good
        best, best_key = -1, None
        for r in range(num_ranks):
            if len(rank_items[r]) >= per:
                continue
            key = (rank_load[r], e in rank_items[r], r)
            if best_key is None or key < best_key:
                best, best_key = r, key
        rank_items[best].append(e)
        rank_load[best] += w
    out = torch.empty(num_physical, dtype=torch.int64)
    for r in range(num_ranks):
        want = list(rank_items[r])
        slots: list[Optional[int]] = [None] * per
        if old_phy2log is not None:
            old = old_phy2log[r * per:(r + 1) * per].tolist()
            for i, e in enumerate(old):         # experts that stay keep their slot: nothing moves for them
                if e in want:
                    slots[i] = e
                    want.remove(e)
        it = iter(want)
        for i in range(per):
            if slots[i] is None:
                slots[i] = next(it)
        out[r * per:(r + 1) * per] = torch.tensor(slots, dtype=torch.int64)
    return out


def build_maps(phy2log: torch.Tensor, num_logical: int, max_copies: Optional[int] = None):
    """``log2phy [E, max_copies]`` (unused entries repeat the first copy, so any index is a valid slot) and
    ``logcnt [E]``."""
    p = phy2log.tolist()
    copies: list[list[int]] = [[] for _ in range(num_logical)]
    for s, e in enumerate(p):
        copies[e].append(s)
    assert all(copies), "every logical expert needs at least one physical slot"
    width = max_copies or max(len(c) for c in copies)
    assert width >= max(len(c) for c in copies)
    log2phy = torch.tensor([c + [c[0]] * (width - len(c)) for c in copies], dtype=torch.int32)
    logcnt = torch.tensor([len(c) for c in copies], dtype=torch.int32)
    return log2phy, logcnt


def balancedness(load: torch.Tensor, phy2log: torch.Tensor, num_ranks: int) -> float:
    """mean / max of the expected pairs per rank (1.0 = even) when the pairs of an expert are shared equally between
    its copies - the figure upstream logs after a re-placement."""
    E = load.numel()
    cnt = torch.bincount(phy2log, minlength=E).double()
    per_slot = (load.double().cpu() / cnt.clamp(min=1))[phy2log]
    per_rank = per_slot.view(num_ranks, -1).sum(1)
    mx = float(per_rank.max())
    return float(per_rank.mean()) / mx if mx > 0 else 1.0


def plan_moves(old_phy2log: torch.Tensor, new_phy2log: torch.Tensor, num_ranks: int):
    """For every slot whose expert changes: ``(dst_slot, src_slot)`` with ``src_slot`` a slot that held the wanted
    expert under the old placement - one on the destination's own rank when there is one, otherwise the copies of
    the expert are used in turn so that no single owner serves every receiver."""
    P = old_phy2log.numel()
    per = P // num_ranks
    old, new = old_phy2log.tolist(), new_phy2log.tolist()
    holders: dict[int, list[int]] = {}
    for s, e in enumerate(old):
        holders.setdefault(e, []).append(s)
    turn: dict[int, int] = {}
    moves = []
    for s in range(P):
        e = new[s]
        if old[s] == e:
            continue
        src = holders[e]
        local = [x for x in src if x // per == s // per]
        if local:
            moves.append((s, local[0]))
        else:
            k = turn.get(e, 0)
            turn[e] = k + 1
            moves.append((s, src[k % len(src)]))
    return moves


def rearrange_layer(tensors: Sequence[torch.Tensor], old_phy2log: torch.Tensor, new_phy2log: torch.Tensor,
                    group_ranks: Sequence[int], rank_in_group: int, group=None) -> int:
    """Move expert rows so that local slot ``i`` of every tensor in ``tensors`` (each ``[num_local, ...]``) holds the
    expert ``new_phy2log`` names.  Returns the number of rows this rank received from other ranks.  Rows that are
    read (sent or copied locally) are staged first, so a slot can be source and destination in the same round."""
    n = len(group_ranks)
    P = old_phy2log.numel()
    per = P // n
    moves = plan_moves(old_phy2log, new_phy2log, n)
    lo = rank_in_group * per
    mine_dst = [(d, s) for d, s in moves if d // per == rank_in_group]
    mine_src = [(d, s) for d, s in moves if s // per == rank_in_group]
    if not mine_dst and not mine_src:
        return 0
    staged = {s: [t[s - lo].clone() for t in tensors] for s in {s for _, s in mine_src}}
    ops, recv = [], []
    # both sides walk the moves in the same (destination slot) order, so the messages of a pair of ranks match up
    for d, s in moves:
        rd, rs = d // per, s // per
        if rd == rs:
            continue
        if rs == rank_in_group:
            for k, row in enumerate(staged[s]):
                ops.append(dist.P2POp(dist.isend, row, group_ranks[rd], group=group, tag=(d * 16 + k) % 32768))
        elif rd == rank_in_group:
            bufs = [torch.empty_like(t[0]) for t in tensors]
            recv.append((d, bufs))
            for k, b in enumerate(bufs):
                ops.append(dist.P2POp(dist.irecv, b, group_ranks[rs], group=group, tag=(d * 16 + k) % 32768))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    for d, s in mine_dst:
        if s // per == rank_in_group:
            for t, row in zip(tensors, staged[s]):
                t[d - lo].copy_(row)
    for d, bufs in recv:
        for t, b in zip(tensors, bufs):
            t[d - lo].copy_(b)
    return len(recv)


class EplbState:
    """Load window + re-placement schedule for all MoE layers of one model (``layers``: the ``FusedMoE`` modules in
    model order, each with EPLB enabled)."""

    def __init__(self, layers, step_interval: int = 3000, window: int = 1000, log: bool = False):
        self.layers = list(layers)
        self.step_interval, self.window = max(1, int(step_interval)), max(1, int(window))
        self.steps = 0
        self.rearrangements = 0
        self.rows_received = 0
        self.last_balancedness: Optional[tuple] = None      # (before, after), averaged over layers
        self.log = log
        if self.layers:
            dev = self.layers[0].expert_load.device
            E = self.layers[0].num_experts
            self._window = torch.zeros(self.window, len(self.layers), E, dtype=torch.int64, device=dev)

    def step(self) -> bool:
        """Called once per engine step on every rank, between steps.  Returns True when a re-placement ran."""
        if not self.layers:
            return False
        slot = self.steps % self.window
        for i, m in enumerate(self.layers):
            self._window[slot, i].copy_(m.expert_load)
            m.expert_load.zero_()
        self.steps += 1
        if self.steps % self.step_interval != 0:
            return False
        self.rearrange()
        return True

    def global_load(self) -> torch.Tensor:
        """``[layers, E]`` pairs per logical expert over the window, summed over the EP group."""
        load = self._window.sum(0)
        m = self.layers[0]
        if m.ep > 1:
            load = m.ep_group.all_reduce(load)
        return load.cpu()

    def rearrange(self) -> None:
        load = self.global_load()
        before, after = [], []
        for i, m in enumerate(self.layers):
            old = m.phy2log.cpu().to(torch.int64)
            new = rebalance(load[i], m.num_physical, m.ep, old)
            before.append(balancedness(load[i], old, m.ep))
            after.append(balancedness(load[i], new, m.ep))
            self.rows_received += m.apply_placement(new)
        self.rearrangements += 1
        self.last_balancedness = (sum(before) / len(before), sum(after) / len(after))
        if self.log:
            print(f"[eplb] re-placement {self.rearrangements}: balancedness "
                  f"{self.last_balancedness[0]:.3f} -> {self.last_balancedness[1]:.3f}", flush=True)

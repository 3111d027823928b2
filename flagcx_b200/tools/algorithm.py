"""InterOp DSL for cross-cluster collectives.

A workflow is written as a ``with`` block; inside it the module-level
functions add buffers, pipeline counts, refresh functions and operations
for individual ranks, and ``to_xml`` writes one plan file per rank:

    with FlagcxWorkflow("ar", Collective.AllReduce, [], [], world_size=4, clusters=[[0, 1], [2, 3]]):
        bufs = [(init_buffer(r, 0, 2), init_buffer(r, 1, 2), init_buffer(r, 2, 1)) for r in range(4)]
        set_pipeline(1, 0, 1, 0, 1)
        for r in range(4):
            add_opr(r, Stage.PreHomoFunc, 0, {Param.send_buff: BuffRef(bufs[r][0], 0, 2),
                                              Param.recv_buff: BuffRef(bufs[r][2], 0, 1),
                                              Param.count: 1, Param.homo_type: 0,
                                              Param.comm_op: Primitive.ReduceScatter})
            ...
        assert check()
        for r in range(4):
            to_xml(r, "plans")

The names (``FlagcxWorkflow``, ``Stage``, ``Param``, ``BuffRef``, ``Primitive``,
``set_pipeline``, ``set_refresh``, ``add_opr``, ``init_buffer``, ``to_xml``,
``check``) and the XML they produce follow the reference's tool
(flagcx/tools/algorithm.py:1-338, utils.py, schema flagcx/core/c2c_ir.h), so its
scripts run unchanged.  New here is ``check()``: the reference returns True
for everything but ``Custom`` (algorithm.py:274-278); this one executes the
plan on symbolic data - every chunk is a multiset of (rank, chunk) inputs -
and verifies the post-condition of the collective on every rank.

Units: buffer sizes, offsets and counts are in chunks; a chunk is
``total elements / nChunks`` when the plan runs, with ``nChunks`` the size of
the receive buffer.  Buffer types: 0 user send buffer, 1 user receive buffer,
2 scratch.
"""
from __future__ import annotations

import os
from collections import Counter
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple

__all__ = ["Collective", "RedOp", "Primitive", "Stage", "Param", "BuffRef", "DataCond", "FlagcxWorkflow", "set_pipeline",
           "set_refresh", "add_opr", "init_buffer", "get_planner", "to_xml", "check", "explain"]


class Collective(Enum):
    P2P = 0
    Custom = 1
    Broadcast = 2
    Gather = 3
    Scatter = 4
    Reduce = 5
    AllReduce = 6
    AllGather = 7
    ReduceScatter = 8
    AlltoAll = 9
    AlltoAllv = 10
    Nop = 11


class RedOp(Enum):
    sum = 0
    prod = 1
    max = 2
    min = 3
    avg = 4
    nop = 5


class Primitive(Enum):
    P2P = 0
    Custom = 1
    Broadcast = 2
    Gather = 3
    Scatter = 4
    Reduce = 5
    AllReduce = 6
    AllGather = 7
    ReduceScatter = 8
    AlltoAll = 9
    AlltoAllv = 10
    Nop = 11
    LocCpy = 12
    LocRed = 13


class Stage(Enum):
    PreHomoFunc = 0
    HeteroFunc = 1
    HomoInterFunc = 2
    PostHomoFunc = 3


class Param(Enum):
    rank = 0
    peer_or_root_rank = 1
    send_type = 2
    recv_type = 3
    send_offset = 4
    recv_offset = 5
    count = 6
    homo_type = 7
    comm_op = 8
    send_buff = 9
    recv_buff = 10
    sub_step = 11


# DataCond[rank][index] = (redop, [input ids]); input id = rank * nchunks + index
DataCond = List[List[Tuple[RedOp, List[int]]]]

_stack: List["FlagcxWorkflow"] = []


def _curr() -> "FlagcxWorkflow":
    if not _stack:
        raise RuntimeError("no FlagcxWorkflow is open (use it in a `with` block)")
    return _stack[-1]


class BuffRef:
    """``count`` chunks starting at ``offset`` of the buffer with id ``bid``."""

    def __init__(self, bid_: int = -1, offset_: int = -1, count_: int = -1):
        self.bid, self.offset, self.count = bid_, offset_, count_

    def buffer(self):
        return _curr().buffers[self.bid]

    def is_valid(self) -> bool:
        return self.bid >= 0 and self.offset >= 0 and self.count >= 0


class _Buffer:
    def __init__(self, bid, rank, type_, size):
        self.id, self.rank, self.type, self.size = bid, rank, type_, size


class _HomoFunc:
    def __init__(self, params: Dict):
        sb: Optional[BuffRef] = params.get(Param.send_buff)
        rb: Optional[BuffRef] = params.get(Param.recv_buff)
        self.root_rank = params.get(Param.peer_or_root_rank, -1)
        self.send_type = sb.buffer().type if sb is not None else params.get(Param.send_type, 0)
        self.recv_type = rb.buffer().type if rb is not None else params.get(Param.recv_type, 1)
        self.send_offset = sb.offset if sb is not None else params.get(Param.send_offset, 0)
        self.recv_offset = rb.offset if rb is not None else params.get(Param.recv_offset, 0)
        self.count = params.get(Param.count, 0)
        self.homo_type = params.get(Param.homo_type, 0)
        op = params.get(Param.comm_op, Primitive.Nop)
        self.comm_op = op if isinstance(op, Primitive) else Primitive(op)

    def xml(self, ind):
        p = " " * ind
        q = " " * (ind + 2)
        return (f"{p}<HomoFunc>\n{q}<rootRank>{self.root_rank}</rootRank>\n{q}<sendType>{self.send_type}</sendType>\n"
                f"{q}<recvType>{self.recv_type}</recvType>\n{q}<sendOffset>{self.send_offset}</sendOffset>\n"
                f"{q}<recvOffset>{self.recv_offset}</recvOffset>\n{q}<count>{self.count}</count>\n"
                f"{q}<homoType>{self.homo_type}</homoType>\n{q}<commOp>{self.comm_op.value}</commOp>\n{p}</HomoFunc>\n")


class _P2pOp:
    def __init__(self, rank, peer, offset, count, is_recv):
        self.rank, self.peer, self.offset, self.count, self.is_recv = rank, peer, offset, count, is_recv


class _HeteroFunc:
    def __init__(self):
        self.ops: List[_P2pOp] = []

    def xml(self, ind):
        p = " " * ind
        out = f"{p}<HeteroFunc>\n"
        for o in self.ops:
            a, b = " " * (ind + 2), " " * (ind + 4)
            out += (f"{a}<P2pOp>\n{b}<rank>{o.rank}</rank>\n{b}<peerRank>{o.peer}</peerRank>\n{b}<offset>{o.offset}</offset>\n"
                    f"{b}<count>{o.count}</count>\n{b}<isRecv>{o.is_recv}</isRecv>\n{a}</P2pOp>\n")
        return out + f"{p}</HeteroFunc>\n"


class FlagcxC2cPlanner:
    """The plan of one rank."""

    def __init__(self, rank, n_seq_pre, n_pipe_pre, n_seq_inter, n_pipe_post, n_seq_post):
        self.rank = rank
        self.counts = (n_seq_pre, n_pipe_pre, n_seq_inter, n_pipe_post, n_seq_post)
        self.refresh = (-1, 0, 0, 0, 0, RedOp.sum)
        self.pre_homo_steps: List[List[_HomoFunc]] = []
        self.hetero_steps: List[List[_HeteroFunc]] = []
        self.homo_inter_steps: List[List[_HomoFunc]] = []
        self.post_homo_steps: List[List[_HomoFunc]] = []

    def set_refresh(self, buff_type, start, offset, count, total_count, red_op):
        self.refresh = (buff_type, start, offset, count, total_count, red_op)

    def add_p2p_op(self, hetero: _HeteroFunc, params: Dict):
        peer = params[Param.peer_or_root_rank]
        cnt = params.get(Param.count, 0)
        so, ro = params.get(Param.send_offset, -1), params.get(Param.recv_offset, -1)
        if so is not None and so >= 0:
            hetero.ops.append(_P2pOp(self.rank, peer, so, cnt, 0))
        if ro is not None and ro >= 0:
            hetero.ops.append(_P2pOp(self.rank, peer, ro, cnt, 1))

    def to_xml(self, n_chunks: int) -> str:
        bt, st, off, cnt, tot, rop = self.refresh
        out = "<FlagcxC2cPlanner>\n"
        out += f"  <nChunks>{n_chunks}</nChunks>\n"
        for tag, v in zip(("nSeqPreSteps", "nPipePreSteps", "nSeqInterSteps", "nPipePostSteps", "nSeqPostSteps"), self.counts):
            out += f"  <{tag}>{v}</{tag}>\n"
        out += (f"  <RefreshFunc>\n    <buffType>{bt}</buffType>\n    <start>{st}</start>\n    <offset>{off}</offset>\n"
                f"    <count>{cnt}</count>\n    <totalCount>{tot}</totalCount>\n    <redOp>{rop.value}</redOp>\n  </RefreshFunc>\n")
        for tag, steps in (("PreHomoFuncSteps", self.pre_homo_steps), ("HeteroFuncSteps", self.hetero_steps),
                           ("HomoInterFuncSteps", self.homo_inter_steps), ("PostHomoFuncSteps", self.post_homo_steps)):
            out += f"  <{tag}>\n"
            for step in steps:
                if not step:
                    out += "    <Step/>\n"
                    continue
                out += "    <Step>\n" + "".join(f.xml(6) for f in step) + "    </Step>\n"
            out += f"  </{tag}>\n"
        return out + "</FlagcxC2cPlanner>\n"


class FlagcxWorkflow:
    def __init__(self, name: str, coll: Collective, pre_data: DataCond, post_data: DataCond, world_size: int,
                 clusters: Optional[Sequence[Sequence[int]]] = None, red_op: RedOp = RedOp.sum, root: int = 0):
        self.name, self.coll, self.pre_data, self.post_data, self.world_size = name, coll, pre_data, post_data, world_size
        if clusters is None:
            half = world_size // 2 if world_size % 2 == 0 and world_size > 1 else world_size
            clusters = [list(range(i, min(i + half, world_size))) for i in range(0, world_size, half)]
        self.clusters = [list(c) for c in clusters]
        self.red_op, self.root = red_op, root
        self.buffers: List[_Buffer] = []
        self.planner: List[FlagcxC2cPlanner] = []
        self.errors: List[str] = []

    def __enter__(self):
        _stack.append(self)
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        _stack.pop()
        return False

    def add_buffer(self, rank_, type_, size_) -> int:
        self.buffers.append(_Buffer(len(self.buffers), rank_, type_, size_))
        return len(self.buffers) - 1

    def n_chunks(self, rank: int) -> int:
        sizes = [b.size for b in self.buffers if b.rank == rank and b.type == 1]
        return max(sizes) if sizes else 1

    def to_xml(self, rank: int, file: Optional[str] = None) -> str:
        text = self.planner[rank].to_xml(self.n_chunks(rank))
        if file:
            os.makedirs(os.path.dirname(file) or ".", exist_ok=True)
            with open(file, "w") as f:
                f.write(text)
        return text

    # ------------------------------------------------------------ symbolic execution
    def _cluster_of(self, rank):
        for ci, c in enumerate(self.clusters):
            if rank in c:
                return ci, c.index(rank)
        raise RuntimeError(f"rank {rank} is in no cluster")

    def _group(self, rank, homo_type):
        ci, li = self._cluster_of(rank)
        if homo_type == 1:
            return [c[li] for c in self.clusters if li < len(c)]
        return self.clusters[ci]

    def semantic_check(self) -> bool:
        """Run the plan on symbolic chunks and compare with the collective's definition."""
        self.errors = []
        W = self.world_size
        size = {t: [0] * W for t in (0, 1, 2)}
        for b in self.buffers:
            size[b.type][b.rank] = max(size[b.type][b.rank], b.size)
        n_in = max(size[0]) if max(size[0]) else max(size[1])
        mem = {t: [[Counter() for _ in range(max(size[t][r], 1) + 64)] for r in range(W)] for t in (0, 1, 2)}
        for r in range(W):
            for i in range(size[0][r]):
                mem[0][r][i] = Counter({(r, i): 1})
        if self.pre_data:
            for r in range(W):
                for i, (_, ids) in enumerate(self.pre_data[r]):
                    mem[0][r][i] = Counter({(x // n_in, x % n_in): 1 for x in ids})

        def err(msg):
            self.errors.append(msg)

        # refresh
        for r, pl in enumerate(self.planner):
            bt, st, off, cnt, tot, rop = pl.refresh
            if bt in (1, 2) and rop == RedOp.sum:
                for i in range(st, st + tot):
                    if not (st + off <= i < st + off + cnt):
                        mem[bt][r][i] = Counter()

        def run_homo(step_lists, label):
            nsteps = max((len(pl_steps) for pl_steps in step_lists), default=0)
            for s in range(nsteps):
                depth = max((len(step_lists[r][s]) if s < len(step_lists[r]) else 0) for r in range(W))
                for k in range(depth):
                    done = set()
                    for r in range(W):
                        if r in done or s >= len(step_lists[r]) or k >= len(step_lists[r][s]):
                            continue
                        f = step_lists[r][s][k]
                        grp = self._group(r, f.homo_type)
                        funcs = {}
                        for m in grp:
                            if s < len(step_lists[m]) and k < len(step_lists[m][s]):
                                funcs[m] = step_lists[m][s][k]
                        if set(funcs) != set(grp):
                            err(f"{label} step {s}.{k}: ranks {sorted(set(grp) - set(funcs))} of the group do not take part")
                            done |= set(grp)
                            continue
                        ops = {fm.comm_op for fm in funcs.values()}
                        cnts = {fm.count for fm in funcs.values()}
                        if len(ops) != 1 or len(cnts) != 1:
                            err(f"{label} step {s}.{k}: group {grp} disagrees on operation or count")
                            done |= set(grp)
                            continue
                        op, c, g = f.comm_op, f.count, len(grp)
                        src = {m: [mem[funcs[m].send_type][m][funcs[m].send_offset + i].copy() for i in range(c * (g if op in (Primitive.ReduceScatter, Primitive.Scatter, Primitive.AlltoAll) else 1))]
                               for m in grp}

                        def put(m, i, val):
                            mem[funcs[m].recv_type][m][funcs[m].recv_offset + i] = val
                        if op == Primitive.AllReduce:
                            for i in range(c):
                                tot_ = sum((src[m][i] for m in grp), Counter())
                                for m in grp:
                                    put(m, i, tot_.copy())
                        elif op == Primitive.ReduceScatter:
                            for kk, m in enumerate(grp):
                                for i in range(c):
                                    put(m, i, sum((src[q][kk * c + i] for q in grp), Counter()))
                        elif op == Primitive.AllGather:
                            for m in grp:
                                for kk, q in enumerate(grp):
                                    for i in range(c):
                                        put(m, kk * c + i, src[q][i].copy())
                        elif op == Primitive.Broadcast:
                            root = grp[f.root_rank if f.root_rank >= 0 else 0]
                            for m in grp:
                                for i in range(c):
                                    put(m, i, src[root][i].copy())
                        elif op == Primitive.Reduce:
                            root = grp[f.root_rank if f.root_rank >= 0 else 0]
                            for i in range(c):
                                put(root, i, sum((src[q][i] for q in grp), Counter()))
                        elif op == Primitive.Gather:
                            root = grp[f.root_rank if f.root_rank >= 0 else 0]
                            for kk, q in enumerate(grp):
                                for i in range(c):
                                    put(root, kk * c + i, src[q][i].copy())
                        elif op == Primitive.Scatter:
                            root = grp[f.root_rank if f.root_rank >= 0 else 0]
                            for kk, m in enumerate(grp):
                                for i in range(c):
                                    put(m, i, src[root][kk * c + i].copy())
                        elif op == Primitive.AlltoAll:
                            for kk, m in enumerate(grp):
                                for jj, q in enumerate(grp):
                                    for i in range(c):
                                        put(m, jj * c + i, src[q][kk * c + i].copy())
                        elif op in (Primitive.Nop,):
                            pass
                        else:
                            err(f"{label} step {s}.{k}: operation {op.name} is not modelled")
                        done |= set(grp)

        def run_hetero():
            nsteps = max((len(pl.hetero_steps) for pl in self.planner), default=0)
            for s in range(nsteps):
                depth = max((len(pl.hetero_steps[s]) if s < len(pl.hetero_steps) else 0) for pl in self.planner)
                for k in range(depth):
                    sends, recvs = {}, {}
                    for r, pl in enumerate(self.planner):
                        if s >= len(pl.hetero_steps) or k >= len(pl.hetero_steps[s]):
                            continue
                        for o in pl.hetero_steps[s][k].ops:
                            (recvs if o.is_recv else sends).setdefault((o.peer, r) if o.is_recv else (r, o.peer), []).append(o)
                    for pair in set(sends) | set(recvs):
                        a, b = sends.get(pair, []), recvs.get(pair, [])
                        if len(a) != len(b):
                            err(f"hetero step {s}.{k}: {len(a)} sends but {len(b)} receives between ranks {pair[0]} -> {pair[1]}")
                            continue
                        staged = []
                        for so, ro in zip(a, b):
                            if so.count != ro.count:
                                err(f"hetero step {s}.{k}: send of {so.count} chunks meets receive of {ro.count} ({pair[0]} -> {pair[1]})")
                                continue
                            staged.append((ro, [mem[1][pair[0]][so.offset + i].copy() for i in range(so.count)]))
                        for ro, vals in staged:
                            for i, v in enumerate(vals):
                                mem[1][pair[1]][ro.offset + i] = v

        run_homo([pl.pre_homo_steps for pl in self.planner], "pre")
        run_hetero()
        run_homo([pl.homo_inter_steps for pl in self.planner], "inter")
        run_homo([pl.post_homo_steps for pl in self.planner], "post")

        # ---- post-condition
        def want(r, i):
            n_out = size[1][r]
            if self.coll == Collective.AllReduce:
                return Counter({(q, i): 1 for q in range(W)})
            if self.coll == Collective.ReduceScatter:
                return Counter({(q, r * n_out + i): 1 for q in range(W)})
            if self.coll == Collective.AllGather:
                per = n_out // W
                return Counter({(i // per, i % per): 1})
            if self.coll == Collective.Broadcast:
                return Counter({(self.root, i): 1})
            if self.coll == Collective.Reduce:
                return Counter({(q, i): 1 for q in range(W)}) if r == self.root else None
            if self.coll == Collective.AlltoAll:
                per = n_out // W
                return Counter({(i // per, r * per + i % per): 1})
            if self.coll == Collective.Custom and self.post_data:
                _, ids = self.post_data[r][i]
                return Counter({(x // n_in, x % n_in): 1 for x in ids})
            return None
        for r in range(W):
            for i in range(size[1][r]):
                w = want(r, i)
                if w is not None and mem[1][r][i] != w:
                    got = dict(mem[1][r][i])
                    err(f"rank {r} receive chunk {i}: holds {got}, expected {dict(w)}")
        return not self.errors


# ---------------------------------------------------------------- module-level helpers

def set_pipeline(n_seq_pre_: int, n_pipe_pre_: int, n_seq_inter_: int, n_pipe_post_: int, n_seq_post_: int):
    w = _curr()
    w.planner = [FlagcxC2cPlanner(r, n_seq_pre_, n_pipe_pre_, n_seq_inter_, n_pipe_post_, n_seq_post_) for r in range(w.world_size)]


def set_refresh(rank_: int, buff_type_: int, start_: int, offset_: int, count_: int, total_count_: int, red_op_: RedOp):
    _curr().planner[rank_].set_refresh(buff_type_, start_, offset_, count_, total_count_, red_op_)


def add_opr(rank_: int, stage_: Stage, step_: int, params_: Optional[Dict]):
    pl = _curr().planner[rank_]
    if stage_ == Stage.HeteroFunc:
        steps = pl.hetero_steps
        while len(steps) <= step_:
            steps.append([])
        if params_ is not None:
            sub = params_.get(Param.sub_step, 0)
            while len(steps[step_]) <= sub:
                steps[step_].append(_HeteroFunc())
            pl.add_p2p_op(steps[step_][sub], params_)
        return
    steps = {Stage.PreHomoFunc: pl.pre_homo_steps, Stage.HomoInterFunc: pl.homo_inter_steps,
             Stage.PostHomoFunc: pl.post_homo_steps}.get(stage_)
    if steps is None:
        raise RuntimeError("Instruction not supported")
    while len(steps) <= step_:
        steps.append([])
    if params_ is not None:
        steps[step_].append(_HomoFunc(params_))


def init_buffer(rank_: int, type_: int, size_: int) -> int:
    return _curr().add_buffer(rank_, type_, size_)


def get_planner(rank_: int) -> FlagcxC2cPlanner:
    if rank_ >= len(_curr().planner):
        raise RuntimeError(f"No planner for rank {rank_}")
    return _curr().planner[rank_]


def to_xml(rank_: int = 0, path_: str = "") -> str:
    w = _curr()
    return w.to_xml(rank=rank_, file=os.path.join(path_, f"{w.name}_{rank_}.xml") if path_ else None)


def check() -> bool:
    return _curr().semantic_check()


def explain() -> List[str]:
    """Messages of the last ``check()`` that failed."""
    return list(_curr().errors)

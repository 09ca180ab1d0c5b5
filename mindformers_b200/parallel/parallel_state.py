"""Process-group algebra: orthogonal TP / CP / EP / DP / PP groups over ``torch.distributed``.

Extends the scheme of the reference's ``parallel_core/inference/parallel_state.py``
(``RankGenerator`` :88-227, ``initialize_model_parallel`` :230-351, order string "tp-dp-pp") with
context and expert parallelism for training. Ranks are laid out with the first token of ``order``
varying fastest, so tensor-parallel peers are neighbouring GPUs. Expert groups re-factor the
``tp·cp·dp`` ranks of one pipeline stage as ``expert_tp · ep · expert_dp``.

Without an initialised process group (single process) every size is 1 and every rank is 0.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


class RankGenerator:
    """Enumerate the rank lists of any combination of parallel dimensions."""

    def __init__(self, tp: int, ep: int, dp: int, pp: int, cp: int, order: str = "tp-cp-ep-dp-pp",
                 rank_offset: int = 0):
        self.sizes = {"tp": tp, "ep": ep, "dp": dp, "pp": pp, "cp": cp}
        order = order.lower()
        names = order.split("-")
        for name, size in self.sizes.items():
            if name not in names:
                if size != 1:
                    raise ValueError(f"dimension {name!r} has size {size} but is missing from order {order!r}")
                names.append(name)
        if len(set(names)) != len(names):
            raise ValueError(f"order {order!r} repeats a dimension")
        self.order = names
        self.world_size = tp * ep * dp * pp * cp
        self.rank_offset = rank_offset

    def get_ranks(self, token: str) -> List[List[int]]:
        """Rank lists of the groups spanning the dimensions in ``token`` (e.g. ``"tp"``, ``"tp-dp"``)."""
        want = token.lower().split("-")
        for w in want:
            if w not in self.sizes:
                raise ValueError(f"unknown parallel dimension {w!r}")
        shape = [self.sizes[n] for n in self.order]
        strides, acc = [], 1
        for s in shape:
            strides.append(acc)
            acc *= s
        in_idx = [i for i, n in enumerate(self.order) if n in want]
        out_idx = [i for i, n in enumerate(self.order) if n not in want]
        groups = []
        for outer in itertools.product(*[range(shape[i]) for i in reversed(out_idx)]):
            base = sum(c * strides[i] for c, i in zip(outer, reversed(out_idx)))
            ranks = []
            for inner in itertools.product(*[range(shape[i]) for i in reversed(in_idx)]):
                ranks.append(self.rank_offset + base + sum(c * strides[i] for c, i in zip(inner, reversed(in_idx))))
            groups.append(sorted(ranks))
        groups.sort(key=lambda g: g[0])
        return groups


@dataclass
class _Group:
    ranks: List[int] = field(default_factory=lambda: [0])
    group: Optional[object] = None

    @property
    def size(self) -> int:
        return len(self.ranks)

    def rank_in_group(self, global_rank: int) -> int:
        return self.ranks.index(global_rank)


class ParallelState:
    """Holds the groups of this rank. Module-level helpers below read the global instance."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.initialized = False
        self.rank = 0
        self.world_size = 1
        self.groups: Dict[str, _Group] = {}
        self.sizes = dict(tp=1, cp=1, ep=1, dp=1, pp=1, etp=1, edp=1)
        self.virtual_pp_size: Optional[int] = None
        self.virtual_pp_rank: Optional[int] = None
        self.rank_lists: Dict[str, list] = {}       # name -> the rank lists of every group of that kind in the job
        self.subgroups: Dict[tuple, tuple] = {}

    def get(self, name: str) -> _Group:
        return self.groups.get(name) or _Group([self.rank])


_STATE = ParallelState()


def _new_group(ranks: Sequence[int], backend=None, timeout=None):
    kwargs = {}
    if backend is not None:
        kwargs["backend"] = backend
    if timeout is not None:
        kwargs["timeout"] = timeout
    return dist.new_group(ranks=list(ranks), **kwargs)


def initialize_model_parallel(tensor_model_parallel_size: int = 1, pipeline_model_parallel_size: int = 1,
                              context_parallel_size: int = 1, expert_model_parallel_size: int = 1,
                              expert_tensor_parallel_size: Optional[int] = None,
                              data_parallel_size: Optional[int] = None,
                              virtual_pipeline_model_parallel_size: Optional[int] = None,
                              order: str = "tp-cp-ep-dp-pp", timeout=None) -> ParallelState:
    """Create every process group. Must be called by all ranks with the same arguments."""
    st = _STATE
    st.reset()
    tp, pp, cp, ep = (tensor_model_parallel_size, pipeline_model_parallel_size, context_parallel_size,
                      expert_model_parallel_size)
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()
    else:
        world, rank = 1, 0
    if world % (tp * pp * cp) != 0:
        raise ValueError(f"world size {world} is not divisible by tp*pp*cp = {tp * pp * cp}")
    dp = world // (tp * pp * cp)
    if data_parallel_size not in (None, dp):
        raise ValueError(f"data_parallel_size {data_parallel_size} does not match world/(tp*pp*cp) = {dp}")
    etp = expert_tensor_parallel_size or tp
    stage = tp * cp * dp
    if stage % (etp * ep) != 0:
        raise ValueError(f"tp*cp*dp = {stage} is not divisible by expert_tp*ep = {etp * ep}")
    edp = stage // (etp * ep)
    st.rank, st.world_size = rank, world
    st.sizes = dict(tp=tp, cp=cp, ep=ep, dp=dp, pp=pp, etp=etp, edp=edp)
    st.virtual_pp_size = virtual_pipeline_model_parallel_size
    st.virtual_pp_rank = 0 if virtual_pipeline_model_parallel_size else None

    dense = RankGenerator(tp=tp, ep=1, dp=dp, pp=pp, cp=cp, order=order)
    expert = RankGenerator(tp=etp, ep=ep, dp=edp, pp=pp, cp=1, order=order)
    plan = {
        "tp": dense.get_ranks("tp"), "cp": dense.get_ranks("cp"), "dp": dense.get_ranks("dp"),
        "pp": dense.get_ranks("pp"), "dp_cp": dense.get_ranks("dp-cp"), "tp_cp": dense.get_ranks("tp-cp"),
        "mp": dense.get_ranks("tp-pp"), "tp_dp_cp": dense.get_ranks("tp-dp-cp"),
        "ep": expert.get_ranks("ep"), "etp": expert.get_ranks("tp"), "edp": expert.get_ranks("dp"),
        "etp_ep": expert.get_ranks("tp-ep"),
    }
    st.rank_lists = {name: [list(r) for r in lists] for name, lists in plan.items()}
    for name, lists in plan.items():
        mine = None
        for ranks in lists:
            grp = _new_group(ranks, timeout=timeout) if world > 1 else None
            if rank in ranks:
                mine = _Group(list(ranks), grp)
        st.groups[name] = mine or _Group([rank])
    st.groups["world"] = _Group(list(range(world)), dist.group.WORLD if world > 1 else None)
    st.initialized = True
    return st


def split_group(name: str, inner: int):
    """Two-level split of the groups called ``name``: ``inner`` consecutive members form an inner group (the ranks of one
    node, say) and the members with the same position inside their inner group form an outer group. Returns
    ``(inner_group, inner_ranks, outer_group, outer_ranks)`` for this rank; process-group handles are ``None`` for
    single-member groups. Every rank of the job must call this with the same arguments (groups are created
    collectively), and the result is cached."""
    st = _STATE
    key = (name, inner)
    if key in st.subgroups:
        return st.subgroups[key]
    lists = st.rank_lists.get(name) or [[st.rank]]
    mine = [None, [st.rank], None, [st.rank]]
    for ranks in lists:
        n = len(ranks)
        if n % inner:
            raise ValueError(f"group {name!r} of size {n} cannot be split into inner groups of {inner}")
        inners = [ranks[i:i + inner] for i in range(0, n, inner)]
        outers = [ranks[i::inner] for i in range(inner)]
        for slot, groups in ((0, inners), (2, outers)):
            for g in groups:
                handle = _new_group(g) if (st.world_size > 1 and len(g) > 1) else None
                if st.rank in g:
                    mine[slot], mine[slot + 1] = handle, list(g)
    st.subgroups[key] = tuple(mine)
    return st.subgroups[key]


def destroy_model_parallel():
    _STATE.reset()


def model_parallel_is_initialized() -> bool:
    return _STATE.initialized


def get_state() -> ParallelState:
    return _STATE


def _size(name):
    return _STATE.get(name).size


def _rank(name):
    g = _STATE.get(name)
    return g.rank_in_group(_STATE.rank)


def get_group(name: str):
    """torch process group handle of ``name`` (None when it has a single member)."""
    return _STATE.get(name).group


def get_group_ranks(name: str) -> List[int]:
    return list(_STATE.get(name).ranks)


def get_tensor_model_parallel_group(): return get_group("tp")
def get_tensor_model_parallel_world_size(): return _size("tp")
def get_tensor_model_parallel_rank(): return _rank("tp")
def get_data_parallel_group(with_context_parallel: bool = False): return get_group("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_world_size(with_context_parallel: bool = False): return _size("dp_cp" if with_context_parallel else "dp")
def get_data_parallel_rank(with_context_parallel: bool = False): return _rank("dp_cp" if with_context_parallel else "dp")
def get_context_parallel_group(): return get_group("cp")
def get_context_parallel_world_size(): return _size("cp")
def get_context_parallel_rank(): return _rank("cp")
def get_pipeline_model_parallel_group(): return get_group("pp")
def get_pipeline_model_parallel_world_size(): return _size("pp")
def get_pipeline_model_parallel_rank(): return _rank("pp")
def get_expert_model_parallel_group(): return get_group("ep")
def get_expert_model_parallel_world_size(): return _size("ep")
def get_expert_model_parallel_rank(): return _rank("ep")
def get_expert_tensor_parallel_group(): return get_group("etp")
def get_expert_tensor_parallel_world_size(): return _size("etp")
def get_expert_tensor_parallel_rank(): return _rank("etp")
def get_expert_data_parallel_group(): return get_group("edp")
def get_expert_data_parallel_world_size(): return _size("edp")
def get_expert_data_parallel_rank(): return _rank("edp")
def get_model_parallel_group(): return get_group("mp")
def get_world_group(): return get_group("world")


def is_pipeline_first_stage(ignore_virtual: bool = False) -> bool:
    if not ignore_virtual and _STATE.virtual_pp_size and _STATE.virtual_pp_rank != 0:
        return False
    return get_pipeline_model_parallel_rank() == 0


def is_pipeline_last_stage(ignore_virtual: bool = False) -> bool:
    if not ignore_virtual and _STATE.virtual_pp_size and _STATE.virtual_pp_rank != _STATE.virtual_pp_size - 1:
        return False
    return get_pipeline_model_parallel_rank() == get_pipeline_model_parallel_world_size() - 1


def get_pipeline_model_parallel_next_rank() -> int:
    g = _STATE.get("pp")
    return g.ranks[(g.rank_in_group(_STATE.rank) + 1) % g.size]


def get_pipeline_model_parallel_prev_rank() -> int:
    g = _STATE.get("pp")
    return g.ranks[(g.rank_in_group(_STATE.rank) - 1) % g.size]


def set_virtual_pipeline_model_parallel_rank(rank: Optional[int]):
    _STATE.virtual_pp_rank = rank


def get_virtual_pipeline_model_parallel_rank(): return _STATE.virtual_pp_rank
def get_virtual_pipeline_model_parallel_world_size(): return _STATE.virtual_pp_size


@dataclass
class ModelCommProcessGroups:
    """Bundle of groups handed to a model (reference ``process_group_config.py:25-123``)."""
    tp: object = None
    dp: object = None
    pp: object = None
    cp: object = None
    ep: object = None
    etp: object = None
    globals: object = None

    @classmethod
    def use_parallel_state_groups(cls, required: Optional[List[str]] = None) -> "ModelCommProcessGroups":
        names = required or ["tp", "dp", "pp", "cp", "ep", "etp"]
        out = cls()
        for n in names:
            setattr(out, n, get_group(n))
        out.globals = get_group("world")
        return out

    @classmethod
    def get_default_model_comm_pgs(cls) -> "ModelCommProcessGroups":
        return cls()

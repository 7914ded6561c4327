"""Process-group topology for mixed DP / TP / Ulysses-CP training plus encoder ranks.

Rank layout (identical to the reference so converted checkpoints and batch semantics
carry over, ``teletron/core/parallel_state.py:299-302, 348-357, 378-379, 468-471``):

* DiT ranks are ``0 .. dit_world-1``; encoder-service ranks sit at the tail.
* Inside the DiT world: tensor-parallel fastest, then context-parallel, then
  data-parallel.  ``rank = dp * (tp*cp) + cp_idx * tp + tp_idx``.

Differences from the reference, on purpose:

* Every rank of the job (encoder ranks included) walks the *same* deterministic list
  of ``new_group`` calls.  The reference creates caller-dependent groups and lets
  encoder ranks skip ~20 creations (``parallel_state.py:130-135, 162-167``), which is
  only safe by accident of the store implementation.
* No patching of ``torch.distributed`` defaults (``parallel_state.py:39-86``): callers
  get explicit group handles.
* Works un-initialised: with no process group every size is 1 and every group ``None``,
  so single-process runs need no ``torch.distributed`` at all.
"""

from __future__ import annotations

import dataclasses
import datetime
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


@dataclasses.dataclass
class CommPair:
    """One encoder-rank -> DiT-rank stream (``parallel_state.py:27-32``).

    ``lane`` / ``lanes``: when there are more encoder ranks than consumers, a consumer is fed by ``lanes`` producers in
    turn; this pair carries the samples whose sequence number is ``lane`` modulo ``lanes``."""
    producer: int
    consumer: int
    dp_rank: int
    dp_size: int
    lane: int = 0
    lanes: int = 1
    group: Optional[object] = dataclasses.field(default=None, compare=False, repr=False)   # two-rank process group of this stream


@dataclasses.dataclass
class _State:
    world_size: int = 1
    rank: int = 0
    dit_world_size: int = 1
    encoder_world_size: int = 0
    tp: int = 1
    cp: int = 1
    dp: int = 1
    tp_rank: int = 0
    cp_rank: int = 0
    dp_rank: int = 0
    is_dit_rank: bool = True
    backend: Optional[str] = None
    world_group: Optional[dist.ProcessGroup] = None
    dit_group: Optional[dist.ProcessGroup] = None
    tp_group: Optional[dist.ProcessGroup] = None
    cp_group: Optional[dist.ProcessGroup] = None
    dp_group: Optional[dist.ProcessGroup] = None
    dp_cp_group: Optional[dist.ProcessGroup] = None
    dp_cp_group_gloo: Optional[dist.ProcessGroup] = None
    tp_cp_group: Optional[dist.ProcessGroup] = None
    tp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    cp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    dp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    dp_cp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    tp_cp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    comm_pairs: List[CommPair] = dataclasses.field(default_factory=list)
    initialized: bool = False
    # pipeline / expert / virtual-pipeline plumbing (groups only: the DiT itself keeps every block on every rank)
    pp: int = 1
    ep: int = 1
    pp_rank: int = 0
    vpp_size: Optional[int] = None
    vpp_rank: Optional[int] = None
    pp_split_rank: Optional[int] = None
    pp_group: Optional[dist.ProcessGroup] = None
    pp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    embd_group: Optional[dist.ProcessGroup] = None
    embd_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    pos_embd_group: Optional[dist.ProcessGroup] = None
    pos_embd_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    mp_group: Optional[dist.ProcessGroup] = None
    mp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    tp_dp_cp_group: Optional[dist.ProcessGroup] = None
    tp_dp_cp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    tp_dp_group: Optional[dist.ProcessGroup] = None
    tp_dp_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    tp_ep_group: Optional[dist.ProcessGroup] = None
    tp_ep_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    ep_group: Optional[dist.ProcessGroup] = None
    ep_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])
    dp_mod_ep_group: Optional[dist.ProcessGroup] = None
    dp_mod_ep_ranks: List[int] = dataclasses.field(default_factory=lambda: [0])


_STATE = _State()


def rank_coords(rank: int, tp: int, cp: int, pp: int = 1, dit_world: Optional[int] = None) -> Dict[str, int]:
    """Coordinates of a DiT rank: tp fastest, then cp, then dp, pipeline stage slowest."""
    stage = 0
    if pp > 1:
        per_stage = dit_world // pp
        stage, rank = rank // per_stage, rank % per_stage
    return {"tp": rank % tp, "cp": (rank // tp) % cp, "dp": rank // (tp * cp), "pp": stage}


def build_rank_lists(dit_world: int, tp: int, cp: int, pp: int = 1, ep: int = 1,
                     pp_split_rank: Optional[int] = None) -> Dict[str, List[List[int]]]:
    """All group memberships as plain lists (pure function; unit-testable without dist).

    With ``pp > 1`` the world is ``pp`` consecutive stages of ``dit_world / pp`` ranks, each laid out as above (the order
    of ``teletron/core/parallel_state.py:299-302, 386-395``).  Besides the five kinds the model uses, the lists cover the
    groups the reference builds for pipeline and expert parallelism (``:386-430``, ``:478-515``): ``pp`` (one rank per
    stage), ``embd`` / ``pos_embd`` (first [+ split] + last stage / first [+ split]), ``mp`` (tensor x pipeline),
    ``tp_dp_cp`` / ``tp_dp``, ``tp_ep`` / ``ep`` / ``dp_mod_ep``."""
    if dit_world % (tp * cp * pp) != 0:
        raise ValueError(f"DiT world size {dit_world} is not divisible by tp*cp*pp = {tp}*{cp}*{pp}")
    per_stage = dit_world // pp
    dp = per_stage // (tp * cp)
    if dp % ep:
        raise ValueError(f"data-parallel size {dp} is not divisible by the expert-parallel size {ep}")
    block = tp * cp
    out: Dict[str, List[List[int]]] = {k: [] for k in ("tp", "cp", "dp", "dp_cp", "tp_cp", "tp_dp_cp", "tp_dp", "tp_ep", "ep",
                                                        "dp_mod_ep")}
    for st in range(pp):
        o = st * per_stage
        out["tp"] += [[o + i * tp + t for t in range(tp)] for i in range(per_stage // tp)]
        out["cp"] += [[o + d * block + c * tp + t for c in range(cp)] for d in range(dp) for t in range(tp)]
        out["dp"] += [[o + d * block + j for d in range(dp)] for j in range(block)]
        # data-parallel "with context parallel": all ranks of the stage sharing a tp index
        out["dp_cp"] += [[o + d * block + c * tp + t for d in range(dp) for c in range(cp)] for t in range(tp)]
        out["tp_cp"] += [list(range(o + d * block, o + (d + 1) * block)) for d in range(dp)]
        out["tp_dp_cp"].append(list(range(o, o + per_stage)))
        out["tp_dp"] += [[o + d * block + c * tp + t for d in range(dp) for t in range(tp)] for c in range(cp)]
        # expert parallelism lives inside data parallelism (cp = 1 in the reference's arithmetic; here per cp index)
        for c in range(cp):
            for e0 in range(0, dp, ep):
                members = [o + d * block + c * tp + t for d in range(e0, e0 + ep) for t in range(tp)]
                out["tp_ep"].append(members)
                out["ep"] += [members[t::tp] for t in range(tp)]
            for j in range(tp * ep):
                d0, t = divmod(j, tp)
                out["dp_mod_ep"].append([o + d * block + c * tp + t for d in range(d0, dp, ep)])
    out["pp"] = [[st * per_stage + i for st in range(pp)] for i in range(per_stage)]
    out["embd"], out["pos_embd"] = [], []
    for ranks in out["pp"]:
        if len(ranks) > 1:
            e, pe = [ranks[0], ranks[-1]], [ranks[0]]
            if pp_split_rank is not None:
                if ranks[pp_split_rank] not in e:
                    e = [ranks[0], ranks[pp_split_rank], ranks[-1]]
                if ranks[pp_split_rank] not in pe:
                    pe = [ranks[0], ranks[pp_split_rank]]
        else:
            e, pe = list(ranks), list(ranks)
        out["embd"].append(e)
        out["pos_embd"].append(pe)
    # model parallel = tensor x pipeline: ranks sharing (dp, cp)
    out["mp"] = [[st * per_stage + d * block + c * tp + t for st in range(pp) for t in range(tp)]
                 for d in range(dp) for c in range(cp)]
    return out


def load_nccl_communicator_config(path: Optional[str]) -> dict:
    """``--nccl-communicator-config-path``: a YAML file ``{group kind: {cga_cluster_size, max_ctas, min_ctas}}`` with the
    kinds ``tp, cp, dp, dp_cp, tp_cp, pp, embd, mp, tp_dp_cp, tp_dp, tp_ep, ep, dp_mod_ep`` (Megatron's file format,
    ``parallel_state.py:279-290``)."""
    if not path:
        return {}
    import yaml
    with open(path) as f:
        return yaml.safe_load(f) or {}


def nccl_options(kind: str, cfgs: dict, backend: Optional[str]):
    """``ProcessGroupNCCL.Options`` carrying the communicator settings configured for this kind of group, or ``None``."""
    if backend != "nccl" or kind not in cfgs:
        return None
    opts = dist.ProcessGroupNCCL.Options()
    c = cfgs[kind] or {}
    opts.config.cga_cluster_size = int(c.get("cga_cluster_size", 4))
    opts.config.max_ctas = int(c.get("max_ctas", 32))
    opts.config.min_ctas = int(c.get("min_ctas", 1))
    return opts


def build_comm_pairs(dit_world: int, encoder_world: int, tp: int, cp: int) -> List[CommPair]:
    """Producer/consumer pairing (``parallel_state.py:174-205``).

    The consumers are the first rank of every TP x CP block (one per data-parallel
    replica); consumer ``i`` is served by encoder rank ``dit_world + i % encoder_world``.
    With more encoder ranks than consumers (the reference would leave the extra ones idle)
    encoder rank ``e`` joins consumer ``e % dp`` and the consumer's samples are dealt out to
    its producers in turn, so the VAE of several encoder GPUs works for one DiT group.
    """
    if encoder_world == 0:
        return []
    block = tp * cp
    dp = dit_world // block
    pairs = []
    if encoder_world <= dp:
        for d in range(dp):
            pairs.append(CommPair(producer=dit_world + d % encoder_world, consumer=d * block, dp_rank=d, dp_size=dp))
        return pairs
    for d in range(dp):
        mine = [e for e in range(encoder_world) if e % dp == d]
        for lane, e in enumerate(mine):
            pairs.append(CommPair(producer=dit_world + e, consumer=d * block, dp_rank=d, dp_size=dp,
                                  lane=lane, lanes=len(mine)))
    return pairs


def _new_group(ranks, backend=None, timeout=None, pg_options=None):
    kwargs = {}
    if timeout is not None:
        kwargs["timeout"] = timeout
    if pg_options is not None:
        kwargs["pg_options"] = pg_options
    return dist.new_group(ranks=ranks, backend=backend, **kwargs)


def initialize_model_parallel(tensor_model_parallel_size: int = 1, context_parallel_size: int = 1,
                              encoder_world_size: int = 0, timeout_minutes: Optional[float] = None,
                              create_gloo_groups: bool = True, pipeline_model_parallel_size: int = 1,
                              virtual_pipeline_model_parallel_size: Optional[int] = None,
                              pipeline_model_parallel_split_rank: Optional[int] = None,
                              expert_model_parallel_size: int = 1,
                              nccl_communicator_config_path: Optional[str] = None) -> None:
    """Create every group.  Must be called by all ranks of the default process group.

    The pipeline / virtual-pipeline / expert arguments build the same extra groups as the reference's
    ``initialize_model_parallel_base`` (``parallel_state.py:386-430, 478-515``); with their defaults no extra group is
    created.  ``nccl_communicator_config_path`` names a YAML file with per-kind NCCL communicator settings."""
    global _STATE
    pp, ep = pipeline_model_parallel_size, expert_model_parallel_size
    if not dist.is_initialized():
        if tensor_model_parallel_size * context_parallel_size * pp * ep != 1 or encoder_world_size:
            raise RuntimeError("torch.distributed is not initialised but parallel sizes > 1 were requested")
        _STATE = _State(initialized=True, vpp_size=virtual_pipeline_model_parallel_size,
                        vpp_rank=0 if virtual_pipeline_model_parallel_size else None)
        return
    world = dist.get_world_size()
    rank = dist.get_rank()
    tp, cp = tensor_model_parallel_size, context_parallel_size
    dit_world = world - encoder_world_size
    if dit_world <= 0:
        raise ValueError("encoder ranks consume the whole world")
    if virtual_pipeline_model_parallel_size is not None and pp <= 2:
        raise ValueError("a virtual (interleaved) pipeline needs pipeline-model-parallel size > 2")
    lists = build_rank_lists(dit_world, tp, cp, pp, ep, pipeline_model_parallel_split_rank)
    timeout = datetime.timedelta(minutes=timeout_minutes) if timeout_minutes else None
    backend = dist.get_backend()
    nccl_cfgs = load_nccl_communicator_config(nccl_communicator_config_path)
    st = _State(world_size=world, rank=rank, dit_world_size=dit_world, encoder_world_size=encoder_world_size,
                tp=tp, cp=cp, dp=dit_world // (tp * cp * pp), is_dit_rank=rank < dit_world, backend=backend, pp=pp, ep=ep,
                vpp_size=virtual_pipeline_model_parallel_size, vpp_rank=0 if virtual_pipeline_model_parallel_size else None,
                pp_split_rank=pipeline_model_parallel_split_rank)
    st.world_group = dist.group.WORLD
    if encoder_world_size > 0:
        st.dit_group = _new_group(list(range(dit_world)), timeout=timeout)
    else:
        st.dit_group = dist.group.WORLD

    def make(kind: str, attr_group: str, attr_ranks: str, gloo_attr: Optional[str] = None):
        for ranks in lists[kind]:
            if len(ranks) == 1:
                # a singleton group needs no communicator; keep the handle None
                if rank in ranks:
                    setattr(st, attr_ranks, ranks)
                continue
            g = _new_group(ranks, timeout=timeout, pg_options=nccl_options(kind, nccl_cfgs, backend))
            g_gloo = _new_group(ranks, backend="gloo", timeout=timeout) if (gloo_attr and create_gloo_groups
                                                                             and backend != "gloo") else None
            if rank in ranks:
                setattr(st, attr_group, g)
                setattr(st, attr_ranks, ranks)
                if gloo_attr:
                    setattr(st, gloo_attr, g_gloo if g_gloo is not None else g)

    make("tp", "tp_group", "tp_ranks")
    make("cp", "cp_group", "cp_ranks")
    make("dp", "dp_group", "dp_ranks")
    make("dp_cp", "dp_cp_group", "dp_cp_ranks", "dp_cp_group_gloo")
    make("tp_cp", "tp_cp_group", "tp_cp_ranks")
    if pp > 1 or ep > 1:
        # same walk on every rank of the job, as for the groups above
        for kind in ("pp", "embd", "pos_embd", "mp", "tp_dp_cp", "tp_dp", "tp_ep", "ep", "dp_mod_ep"):
            make(kind, kind + "_group", kind + "_ranks")
    if st.is_dit_rank:
        c = rank_coords(rank, tp, cp, pp, dit_world)
        st.tp_rank, st.cp_rank, st.dp_rank, st.pp_rank = c["tp"], c["cp"], c["dp"], c["pp"]
    st.comm_pairs = build_comm_pairs(dit_world, encoder_world_size, tp, cp)
    # every stream gets its own two-rank group: point-to-point traffic on the world communicator would be serialised
    # with everything else issued on it (and, with NCCL's eager initialisation, is treated like a collective)
    for pair in st.comm_pairs:
        pair.group = _new_group([pair.consumer, pair.producer], timeout=timeout)
    st.initialized = True
    _STATE = st


def destroy_model_parallel() -> None:
    global _STATE
    _STATE = _State()


def model_parallel_is_initialized() -> bool:
    return _STATE.initialized


def state() -> _State:
    return _STATE


# ---- getters with the reference's public names (parallel_state.py:546-585) -----------------

def get_world_group():
    return _STATE.world_group


def get_transformer_model_group():
    return _STATE.dit_group


def get_tensor_model_parallel_group():
    return _STATE.tp_group


def get_tensor_model_parallel_world_size() -> int:
    return _STATE.tp


def get_tensor_model_parallel_rank() -> int:
    return _STATE.tp_rank


def get_context_parallel_group():
    return _STATE.cp_group


def get_context_parallel_world_size() -> int:
    return _STATE.cp


def get_context_parallel_rank() -> int:
    return _STATE.cp_rank


def get_data_parallel_group(with_context_parallel: bool = False):
    return _STATE.dp_cp_group if with_context_parallel else _STATE.dp_group


def get_data_parallel_group_gloo(with_context_parallel: bool = True):
    return _STATE.dp_cp_group_gloo


def get_data_parallel_world_size(with_context_parallel: bool = False) -> int:
    return _STATE.dp * _STATE.cp if with_context_parallel else _STATE.dp


def get_data_parallel_rank(with_context_parallel: bool = False) -> int:
    if with_context_parallel:
        return _STATE.dp_rank * _STATE.cp + _STATE.cp_rank
    return _STATE.dp_rank


def get_data_parallel_ranks(with_context_parallel: bool = False) -> List[int]:
    return _STATE.dp_cp_ranks if with_context_parallel else _STATE.dp_ranks


def get_tensor_context_parallel_group():
    return _STATE.tp_cp_group


def get_tensor_context_parallel_world_size() -> int:
    return _STATE.tp * _STATE.cp


def get_tensor_context_parallel_rank() -> int:
    return _STATE.cp_rank * _STATE.tp + _STATE.tp_rank


def get_tensor_context_parallel_src_rank() -> int:
    """Global rank of the first member of this rank's TP x CP block."""
    return _STATE.tp_cp_ranks[0]


def is_dit_rank() -> bool:
    return _STATE.is_dit_rank


# ---- pipeline / virtual-pipeline / expert plumbing (Megatron's names; sizes are 1 and groups None unless requested) ----

def get_pipeline_model_parallel_group():
    return _STATE.pp_group


def get_pipeline_model_parallel_world_size() -> int:
    return _STATE.pp


def get_pipeline_model_parallel_rank() -> int:
    return _STATE.pp_rank


def get_pipeline_model_parallel_first_rank() -> int:
    return _STATE.pp_ranks[0]


def get_pipeline_model_parallel_last_rank() -> int:
    return _STATE.pp_ranks[-1]


def get_pipeline_model_parallel_next_rank() -> int:
    r = _STATE.pp_ranks
    return r[(_STATE.pp_rank + 1) % len(r)]


def get_pipeline_model_parallel_prev_rank() -> int:
    r = _STATE.pp_ranks
    return r[(_STATE.pp_rank - 1) % len(r)]


def get_virtual_pipeline_model_parallel_world_size() -> Optional[int]:
    return _STATE.vpp_size


def get_virtual_pipeline_model_parallel_rank() -> Optional[int]:
    return _STATE.vpp_rank


def set_virtual_pipeline_model_parallel_rank(rank: Optional[int]) -> None:
    _STATE.vpp_rank = rank


def is_pipeline_first_stage(ignore_virtual: bool = False) -> bool:
    if not ignore_virtual and _STATE.vpp_size is not None and _STATE.vpp_rank != 0:
        return False
    return _STATE.pp_rank == 0


def is_pipeline_last_stage(ignore_virtual: bool = False) -> bool:
    if not ignore_virtual and _STATE.vpp_size is not None and _STATE.vpp_rank != _STATE.vpp_size - 1:
        return False
    return _STATE.pp_rank == _STATE.pp - 1


def get_embedding_group():
    return _STATE.embd_group


def get_position_embedding_group():
    return _STATE.pos_embd_group


def is_rank_in_embedding_group() -> bool:
    return _STATE.rank in _STATE.embd_ranks


def get_model_parallel_group():
    """Tensor x pipeline ranks that together hold one replica's weights."""
    return _STATE.mp_group if _STATE.pp > 1 else _STATE.tp_group


def get_tensor_and_data_parallel_group(with_context_parallel: bool = False):
    return _STATE.tp_dp_cp_group if with_context_parallel else _STATE.tp_dp_group


def get_expert_model_parallel_group():
    return _STATE.ep_group


def get_expert_model_parallel_world_size() -> int:
    return _STATE.ep


def get_expert_model_parallel_rank() -> int:
    return _STATE.ep_ranks.index(_STATE.rank) if _STATE.rank in _STATE.ep_ranks else 0


def get_tensor_and_expert_parallel_group():
    return _STATE.tp_ep_group


def get_data_modulo_expert_parallel_group():
    return _STATE.dp_mod_ep_group


def get_comm_pairs() -> List[CommPair]:
    return list(_STATE.comm_pairs)


def get_comm_pair() -> Optional[CommPair]:
    """The pair this DiT rank consumes from (None for non-src ranks or without encoder ranks)."""
    for p in _STATE.comm_pairs:
        if p.consumer == _STATE.rank:
            return p
    return None


def get_consumer_pairs() -> List[CommPair]:
    """Every stream this DiT rank consumes from, ordered by lane (empty for non-src ranks)."""
    return sorted((p for p in _STATE.comm_pairs if p.consumer == _STATE.rank), key=lambda p: p.lane)


def get_producer_pairs() -> List[CommPair]:
    """All pairs served by this encoder rank."""
    return [p for p in _STATE.comm_pairs if p.producer == _STATE.rank]


_SINGLE_NODE: Dict[int, bool] = {}


def group_is_single_node(group) -> bool:
    """True when every rank of ``group`` runs on this host, i.e. peer memory can be mapped through CUDA IPC.  The in-kernel
    collectives need that; a group that spans hosts keeps the NCCL path.  Collective on first use per group (cached)."""
    if group is None or not dist.is_initialized():
        return True
    key = id(group)
    if key not in _SINGLE_NODE:
        import socket
        try:
            with open("/proc/sys/kernel/random/boot_id") as f:        # two containers on one host may share a hostname
                ident = socket.gethostname() + ":" + f.read().strip()
        except OSError:
            ident = socket.gethostname()
        names = [None] * dist.get_world_size(group)
        dist.all_gather_object(names, ident, group=group)
        _SINGLE_NODE[key] = len(set(names)) == 1
    return _SINGLE_NODE[key]


def local_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")) % max(torch.cuda.device_count(), 1))
    return torch.device("cpu")

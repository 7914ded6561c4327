"""Pipeline / expert / virtual-pipeline group plumbing and the NCCL communicator config file, on CPU ranks."""

import torch

from dist_utils import run_distributed


def test_rank_lists_partition_the_world_for_every_kind():
    from teletron_b200.parallel.state import build_rank_lists
    W, tp, cp, pp, ep = 32, 2, 2, 2, 2
    L = build_rank_lists(W, tp, cp, pp, ep)
    for kind in ("tp", "cp", "dp", "dp_cp", "tp_cp", "pp", "mp", "tp_dp_cp", "tp_dp", "tp_ep", "ep", "dp_mod_ep"):
        flat = sorted(r for g in L[kind] for r in g)
        assert flat == list(range(W)), kind                      # every rank in exactly one group of each kind
    assert all(len(g) == n for kind, n in (("tp", tp), ("cp", cp), ("dp", 4), ("pp", pp), ("mp", tp * pp), ("ep", ep),
                                           ("tp_ep", tp * ep), ("dp_mod_ep", 2), ("tp_dp", 8), ("tp_dp_cp", 16)) for g in L[kind])
    # a pipeline group holds the same (tp, cp, dp) position of every stage; stages are consecutive blocks of ranks
    assert L["pp"][5] == [5, 21] and L["embd"][5] == [5, 21] and L["pos_embd"][5] == [5]
    # split rank adds the first decoder stage to the embedding groups
    L3 = build_rank_lists(12, 1, 1, 4, 1, pp_split_rank=2)
    assert L3["pp"][0] == [0, 3, 6, 9] and L3["embd"][0] == [0, 6, 9] and L3["pos_embd"][0] == [0, 6]
    # expert parallelism sits inside data parallelism: an ep group shares tp / cp index and stage
    assert [0, 4] in L["ep"] and [0, 1, 4, 5] in L["tp_ep"]


def _groups(rank, world):
    import torch.distributed as dist
    from teletron_b200.parallel import state as ps
    ps.initialize_model_parallel(2, 1, pipeline_model_parallel_size=2, expert_model_parallel_size=2)
    out = {"pp": (ps.get_pipeline_model_parallel_world_size(), ps.get_pipeline_model_parallel_rank(),
                  ps.get_pipeline_model_parallel_next_rank(), ps.get_pipeline_model_parallel_prev_rank()),
           "first_last": (ps.is_pipeline_first_stage(), ps.is_pipeline_last_stage()),
           "dp": ps.get_data_parallel_world_size(), "tp": ps.get_tensor_model_parallel_rank(),
           "ep": (ps.get_expert_model_parallel_world_size(), ps.get_expert_model_parallel_rank())}
    for name, g in (("pp_sum", ps.get_pipeline_model_parallel_group()), ("mp_sum", ps.get_model_parallel_group()),
                    ("ep_sum", ps.get_expert_model_parallel_group()), ("embd_sum", ps.get_embedding_group()),
                    ("tpdp_sum", ps.get_tensor_and_data_parallel_group())):
        t = torch.tensor([float(rank)])
        dist.all_reduce(t, group=g)
        out[name] = float(t)
    ps.destroy_model_parallel()
    return out


def test_pipeline_and_expert_groups_on_eight_ranks():
    res = run_distributed(_groups, 8, timeout=180)
    # tp2 x pp2 x dp2: stage 0 = ranks 0-3, stage 1 = ranks 4-7
    for r, o in enumerate(res):
        stage = r // 4
        assert o["pp"] == (2, stage, (r + 4) % 8, (r + 4) % 8)
        assert o["first_last"] == (stage == 0, stage == 1)
        assert o["dp"] == 2 and o["tp"] == r % 2 and o["ep"][0] == 2
        assert o["pp_sum"] == r % 4 + (r % 4 + 4) == o["embd_sum"]
        mp = [r % 2 ^ 0, 0]   # placeholder to keep the expression below readable
        base = (r % 4) // 2 * 2
        assert o["mp_sum"] == sum([base, base + 1, base + 4, base + 5])
        assert o["ep_sum"] == (r % 2) + (r % 2 + 2) + 2 * 4 * stage
        assert o["tpdp_sum"] == sum(range(4 * stage, 4 * stage + 4))


def test_nccl_communicator_config_file(tmp_path):
    from teletron_b200.parallel import state as ps
    path = tmp_path / "nccl.yaml"
    path.write_text("tp:\n  cga_cluster_size: 2\n  max_ctas: 16\n  min_ctas: 2\ndp_cp: {max_ctas: 8}\n")
    cfg = ps.load_nccl_communicator_config(str(path))
    assert cfg["tp"] == {"cga_cluster_size": 2, "max_ctas": 16, "min_ctas": 2} and cfg["dp_cp"]["max_ctas"] == 8
    assert ps.load_nccl_communicator_config(None) == {}
    assert ps.nccl_options("tp", cfg, "gloo") is None and ps.nccl_options("cp", cfg, "nccl") is None
    if hasattr(torch.distributed, "ProcessGroupNCCL"):
        o = ps.nccl_options("tp", cfg, "nccl")
        assert (o.config.cga_cluster_size, o.config.max_ctas, o.config.min_ctas) == (2, 16, 2)


def test_tp_comm_overlap_selects_the_fused_sequence_parallel_path():
    from teletron_b200.training.args import build_parser, validate_args
    a = validate_args(build_parser().parse_args(["--tensor-model-parallel-size", "2", "--tp-comm-overlap"]), world_size=2)
    assert a.sequence_parallel and a.fused_comm
    b = validate_args(build_parser().parse_args(["--tp-comm-overlap"]), world_size=1)
    assert not b.sequence_parallel

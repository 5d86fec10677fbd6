import pytest

from steptronoss_b200.exp.base_exp import ParallelConfig
from steptronoss_b200.parallel.state import ParallelManager, layout_from_pattern


def test_patterns_tp_pp_dp():
    # world 8, p=2, t=2 -> d=2 ; rank = p*4 + d*2 + t
    tp = layout_from_pattern("(p d t) -> (p d) t", 8, p=2, t=2)
    pp = layout_from_pattern("(p d t) -> (d t) p", 8, p=2, t=2)
    dp = layout_from_pattern("(p d t) -> (p t) d", 8, p=2, t=2)
    assert tp == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert pp == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert dp == [[0, 2], [1, 3], [4, 6], [5, 7]]


def test_patterns_cp_and_ep():
    cp = layout_from_pattern("(p d c t) -> (p d t) c", 8, p=1, c=2, t=2)
    assert cp == [[0, 2], [1, 3], [4, 6], [5, 7]]
    ep = layout_from_pattern("(p edp ep etp) -> (p edp etp) ep", 8, p=1, ep=4, etp=1)
    assert ep == [[0, 1, 2, 3], [4, 5, 6, 7]]
    edp = layout_from_pattern("(p edp ep etp) -> (p ep etp) edp", 8, p=1, ep=4, etp=1)
    assert edp == [[0, 4], [1, 5], [2, 6], [3, 7]]


def test_leftover_row_and_errors():
    rows = layout_from_pattern("(p d t) -> (p d) t", 7, p=1, t=2)
    assert rows[-1] == [6] and rows[0] == [0, 1]
    with pytest.raises(ValueError):
        layout_from_pattern("(p d t) -> (p d) t", 2, p=2, t=2)


@pytest.mark.parametrize("rank", range(8))
def test_manager_any_rank_of_a_mesh(rank):
    pm = ParallelManager()
    pm.world_size, pm.world_rank = 8, rank
    cfg = ParallelConfig()
    cfg.tensor_model_parallel_size = 2
    cfg.pipeline_model_parallel_size = 2
    cfg.expert_tensor_parallel_size = 1
    cfg.expert_model_parallel_size = 2
    import steptronoss_b200.parallel.state as st

    old = st.PM
    st.PM = pm
    try:
        import steptronoss_b200.exp.base_exp  # build_parallel looks PM up at call time
        rows = {}
        for name, pattern in cfg.parallel_definition.items():
            axes = set(pattern.split("->")[0].replace("(", " ").replace(")", " ").split())
            sizes = {"p": 2, "c": 1, "ep": 2, "t": 2, "etp": 1}
            rows[name] = pm.define_parallel(pattern, **{k: v for k, v in sizes.items() if k in axes})
            pm.new_parallel(name, rows[name])
    finally:
        st.PM = old
    assert pm.size_of("TP") == 2 and pm.size_of("PP") == 2 and pm.size_of("DP") == 2
    assert pm.rank_in("TP") == rank % 2 and pm.rank_in("PP") == rank // 4
    assert pm.rank_in("DP") == (rank // 2) % 2
    assert pm.is_pipeline_first_stage() == (rank < 4)
    assert pm.size_of("EP") == 2 and pm.size_of("EDP") == 2


def test_named_rng_streams_differ_across_family():
    import torch

    seeds = []
    for rank in range(2):
        pm = ParallelManager()
        pm.world_size, pm.world_rank = 2, rank
        pm.new_parallel("TP", [[0, 1]])
        pm.register_rng("drop", 100, ["TP"])
        with pm.use_rng("drop"):
            seeds.append(torch.rand(1).item())
        with pm.use_rng("drop"):
            second = torch.rand(1).item()
        assert second != seeds[-1]
    assert seeds[0] != seeds[1]


def test_global_memory_buffer_reuses_and_grows():
    import torch

    from steptronoss_b200.parallel.state import destroy_global_memory_buffer, get_global_memory_buffer

    destroy_global_memory_buffer()
    buf = get_global_memory_buffer()
    assert buf is get_global_memory_buffer()
    a = buf.get_tensor((4, 8), torch.float32, "mpu")
    a.fill_(3.0)
    b = buf.get_tensor((2, 8), torch.float32, "mpu")
    assert b.data_ptr() == a.data_ptr() and float(b.sum()) == 48.0            # same storage, no new allocation
    c = buf.get_tensor((2, 8), torch.bfloat16, "mpu")
    d = buf.get_tensor((2, 8), torch.float32, "other")
    assert c.data_ptr() != a.data_ptr() and d.data_ptr() != a.data_ptr()      # keyed by name and dtype
    big = buf.get_tensor((16, 8), torch.float32, "mpu")
    assert big.shape == (16, 8) and buf.nbytes() == 16 * 8 * 4 + 16 * 2 + 16 * 4
    destroy_global_memory_buffer()
    assert get_global_memory_buffer().nbytes() == 0


def test_free_functions_answer_from_the_manager():
    import steptronoss_b200.parallel.state as st

    pm = ParallelManager()
    pm.world_size, pm.world_rank = 8, 5
    old = st.PM
    st.PM = pm
    try:
        assert st.is_unitialized() and not st.model_parallel_is_initialized()
        for name, pattern, sizes in (("TP", "(p d t) -> (p d) t", {"p": 2, "t": 2}), ("PP", "(p d t) -> (d t) p", {"p": 2, "t": 2}),
                                     ("DP", "(p d t) -> (p t) d", {"p": 2, "t": 2}), ("CP", "(p d c t) -> (p d t) c", {"p": 2, "t": 2, "c": 1})):
            pm.new_parallel(name, pm.define_parallel(pattern, **sizes))
        assert not st.is_unitialized() and st.model_parallel_is_initialized()
        # rank 5 = stage 1, data replica 0, tensor rank 1; its pipeline row is [1, 5]
        assert st.get_pipeline_model_parallel_rank() == 1 and st.get_pipeline_model_parallel_world_size() == 2
        assert st.get_pipeline_model_parallel_next_rank() == 1 and st.get_pipeline_model_parallel_prev_rank() == 1
        assert st.is_pipeline_last_stage() and not st.is_pipeline_first_stage()
        assert (st.get_data_rank(), st.get_data_world_size()) == (0, 2)
        st.set_vpp_size(3)
        st.set_vpp_rank(1)
        assert (st.get_vpp_size(), st.get_vpp_rank()) == (3, 1)
        assert st.get_pipeline_model_parallel_world_size(ignore_virtual=False) == 6
        assert st.get_pipeline_model_parallel_rank(ignore_virtual=False) == 1 * 2 + 1      # chunk 1 of stage 1
        assert not st.is_pipeline_last_stage() and st.is_pipeline_last_stage(ignore_virtual=True)
        st.set_vpp_rank(2)
        assert st.is_pipeline_last_stage()
    finally:
        st.PM = old

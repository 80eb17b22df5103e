"""GPU data-generation kernels against the CPU library (same SplitMix64 stream, so results must be identical)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_gpu_chaos_game_matches_cpu_bit_for_bit():
    from scaffold_b200.data import category_search as cs, ifs
    params = np.stack([cs.propose_params(523, 0, i) for i in range(64)])
    seeds = np.array([cs.orbit_seed(523, 0, i) for i in range(64)], dtype=np.uint64)
    s_cpu = ifs.orbit_stats(params, seeds, 500, device="cpu")
    s_gpu = ifs.orbit_stats(params, seeds, 500, device="cuda")
    finite = np.isfinite(s_cpu).all(1)
    np.testing.assert_array_equal(s_cpu[finite], s_gpu[finite])
    v_cpu, _ = ifs.accept(s_cpu, 1.0, 0.15)
    v_gpu, _ = ifs.accept(s_gpu, 1.0, 0.15)
    np.testing.assert_array_equal(v_cpu, v_gpu)
    p_cpu, f_cpu = ifs.orbit_points(params[:8], seeds[:8], 300, device="cpu")
    p_gpu, f_gpu = ifs.orbit_points(params[:8], seeds[:8], 300, device="cuda")
    np.testing.assert_array_equal(f_cpu & 1, f_gpu & 1)
    ok = f_cpu == 0
    np.testing.assert_array_equal(p_cpu[ok], p_gpu[ok])


def test_gpu_rasteriser_matches_cpu_per_shard():
    from scaffold_b200.data import volumes
    rng = np.random.default_rng(3)
    clouds = [(rng.standard_normal((4000, 3)) * s).astype(np.float32) for s in ([1, .6, .3], [.4, 1, .7], [.8, .8, 1])]
    cats = [0, 2, 1]
    colors = rng.random((3, 3))
    for shards, dims, sid in (([1, 1, 1], [2, 3, 4], 0), ([2, 1, 2], [2, 3, 4], 3), ([1, 2, 1], [2, 3, 4], 1)):
        v_cpu, m_cpu = volumes.render_volume_shard(clouds, cats, colors, 32, shards, dims, sid, "cpu")
        v_gpu, m_gpu = volumes.render_volume_shard(clouds, cats, colors, 32, shards, dims, sid, "cuda")
        np.testing.assert_array_equal(m_cpu, m_gpu)
        np.testing.assert_array_equal(v_cpu, v_gpu)

"""Host-side mirror of the reference interface, exercised without a GPU."""
import pytest
import torch

from trak_b200 import fast_jl, projectors


def test_six_entry_points_exist():
    for t in ("rademacher", "normal"):
        for b in (8, 16, 32):
            assert callable(getattr(fast_jl, f"project_{t}_{b}"))


def test_input_checks_match_reference_error_types():
    # fast_jl.cu:23-27,37 -> RuntimeError; pybind uint32 conversion -> TypeError
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        fast_jl.project_rademacher_8(torch.zeros(8, 100), 512, 0, 148)
    with pytest.raises(RuntimeError):
        fast_jl.project_rademacher_8("nope", 512, 0, 148)


def test_u32_conversion():
    assert fast_jl._u32("seed", 5) == 5
    assert fast_jl._u32("seed", 0xFFFFFFFF) == 0xFFFFFFFF
    for bad in (-1, 1 << 32, 1.5, "3"):
        with pytest.raises(TypeError):
            fast_jl._u32("seed", bad)


def test_projection_type_enum():
    assert projectors.ProjectionType.normal.value == "normal"
    assert projectors.ProjectionType("rademacher") is projectors.ProjectionType.rademacher
    assert projectors._ptype_code(projectors.ProjectionType.normal) == 1
    assert projectors._ptype_code("rademacher") == 0
    with pytest.raises(KeyError):
        projectors._ptype_code("gaussian")


def test_cuda_projector_rejects_cpu_device():
    with pytest.raises(ValueError, match="CUDA device"):
        projectors.CudaProjector(100, 512, 0, projectors.ProjectionType.rademacher, "cpu", 32)


def test_vectorize_layout():
    g = {"w": torch.arange(24.0).reshape(2, 3, 4), "b": torch.tensor([7.0, 8.0]),
         "v": torch.arange(6.0).reshape(2, 3)}
    out = projectors.vectorize(g, device="cpu")
    assert out.shape == (2, 12 + 1 + 3)
    assert torch.equal(out[0], torch.cat([torch.arange(12.0), torch.tensor([7.0]), torch.arange(3.0)]))
    assert torch.equal(out[1, 12], torch.tensor(8.0))


class _FakeProjector:
    """Stands in for a per-chunk projector: 'projects' by summing features, scaled by its seed."""

    def __init__(self, seed, proj_dim=4):
        self.seed, self.proj_dim, self.proj_type = seed, proj_dim, "rademacher"
        self.calls = []

    def project(self, grads, model_id):
        self.calls.append(tuple(grads.shape))
        return grads.float().sum(1, keepdim=True).expand(-1, self.proj_dim) * self.seed


def test_chunked_projector_packs_whole_parameters_and_sums_chunks():
    # three parameters of 6, 1 and 5 features; cap 8 -> chunks [6 + 1, 5]
    grads = {"a": torch.ones(3, 2, 3), "b": torch.full((3,), 2.0), "c": torch.full((3, 5), 3.0)}
    fakes = [_FakeProjector(1), _FakeProjector(10)]
    cp = projectors.ChunkedCudaProjector(fakes, max_chunk_size=8, params_per_chunk=[7, 5], feat_bs=4,
                                         device=torch.device("cpu"), dtype=torch.float32)
    out = cp.project(grads, model_id=0)
    assert out.shape == (3, 4)
    assert fakes[0].calls == [(3, 7)] and fakes[1].calls == [(3, 5)]
    assert torch.equal(out, torch.full((3, 4), (6 + 2) * 1.0 + 15 * 10.0))
    cp.free_memory()
    assert not cp.input_allocated


def test_chunked_projector_detects_inconsistent_chunking():
    grads = {"a": torch.ones(2, 6), "b": torch.ones(2, 6)}
    cp = projectors.ChunkedCudaProjector([_FakeProjector(1), _FakeProjector(1)], max_chunk_size=8,
                                         params_per_chunk=[5, 7], feat_bs=2, device=torch.device("cpu"),
                                         dtype=torch.float32)
    with pytest.raises(AssertionError):
        cp.project(grads, model_id=0)


def test_parameter_chunk_sizes_follow_the_reference_rule():
    # expected values produced by the unmodified trak.utils.get_parameter_chunk_sizes on this model
    m = torch.nn.Sequential(torch.nn.Linear(300, 200), torch.nn.Linear(200, 100), torch.nn.Linear(100, 7))
    want = {50000: (85899, [81007]), 70000: (61356, [60200, 20807]), 200000: (21474, [0, 60000, 21007]),
            2 ** 20: (4095, [0, 60000, 200, 20000, 807])}
    for bs, (cap, sizes) in want.items():
        assert projectors.get_parameter_chunk_sizes(m, bs) == (cap, sizes)
    widths = [p.numel() for p in m.parameters()]
    assert projectors.get_parameter_chunk_sizes(widths, max_chunk_size=61356)[1] == [60200, 20807]
    with pytest.raises(ValueError):
        projectors.get_parameter_chunk_sizes(widths)


def test_chunked_projector_rejects_empty_chunks_and_oversized_batches():
    grads = {"a": torch.ones(2, 9), "b": torch.ones(2, 3)}
    cp = projectors.ChunkedCudaProjector([_FakeProjector(1), _FakeProjector(1), _FakeProjector(1)], max_chunk_size=8,
                                         params_per_chunk=[0, 9, 3], feat_bs=2, device=torch.device("cpu"),
                                         dtype=torch.float32)
    with pytest.raises(ValueError, match="larger than"):
        cp.project(grads, model_id=0)       # the first parameter alone exceeds the cap: empty leading chunk
    cp2 = projectors.ChunkedCudaProjector([_FakeProjector(1)], max_chunk_size=100, params_per_chunk=[12], feat_bs=1,
                                          device=torch.device("cpu"), dtype=torch.float32)
    with pytest.raises(RuntimeError, match="feat_bs"):
        cp2.project(grads, model_id=0)      # two rows into a projector sized for one


def test_finalize_and_featurize_components_need_a_cuda_device():
    from trak_b200.featurize import FeatureWriter
    from trak_b200.finalize import ScoreFinalizer
    with pytest.raises(ValueError):
        ScoreFinalizer([torch.zeros(4, 2)], [torch.zeros(3, 2)], [torch.zeros(4, 1)], "cpu")
    with pytest.raises(ValueError):
        FeatureWriter(_FakeProjector(1), 1.0, torch.float32, "cpu", max_batch=4)


def test_install_fast_jl_shim_registers_the_module(monkeypatch):
    import sys
    import trak_b200
    monkeypatch.delitem(sys.modules, "fast_jl", raising=False)
    trak_b200.install_fast_jl_shim()
    import fast_jl
    assert fast_jl is trak_b200.fast_jl
    for t in ("rademacher", "normal"):
        for b in (8, 16, 32):
            assert callable(getattr(fast_jl, f"project_{t}_{b}"))
    monkeypatch.delitem(sys.modules, "fast_jl", raising=False)

"""The traffic model bench.py reports against: the reference's own byte counts for the int4 GEMMs
(scripts/shape_utils.py:310-321 of the reference), pinned to the figures its documents quote."""

import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_bytes_match_the_reference_model():
    b = _bench()
    assert b.alg_bytes(1, 4096, 4096) == 8_667_136
    assert [b.alg_bytes(m, 28672, 4096) for m in (1, 16, 64)] == [60_620_800, 61_603_840, 64_749_568]
    assert [b.alg_bytes(m, 4096, 14336) for m in (1, 16, 64)] == [30_314_496, 30_867_456, 32_636_928]
    assert b.step_bytes(16) == 16 * (60_620_800 + 61_603_840 + 64_749_568 + 30_314_496 + 30_867_456 + 32_636_928)


def test_default_routes_named_in_the_bench_line():
    b = _bench()
    assert b.kernel_for(1) == "w4_stream_kernel" and b.kernel_for(8) == "w4_stream_kernel"
    assert b.kernel_for(16) == "w4_tmem_kernel" and b.kernel_for(64) == "w4_tmem_kernel"
    assert set(b.NCU_TRAFFIC_RATIO) == {"w4_stream_kernel", "w4_tmem_kernel"}


def test_projection_stack_bytes_match_the_reference_figure():
    """Weights and scales of the full-depth Llama-3-8B int4 stack are the reference's 3.60 GB per pass
    (docs/design/llm_quant.md:184-185); the stack's algorithmic bytes add the bf16 activations and
    outputs of the 64 tokens, and do not depend on the tensor-parallel degree."""
    import sys

    sys.path.insert(0, os.path.join(ROOT, "5090-blackwell-kernels_b200", "python"))
    from spark_kernels import tp

    shape = tp.LlamaShape()
    for degree in (1, 2, 4, 8):
        st = tp.ProjectionStack.__new__(tp.ProjectionStack)
        st.shape, st.M, st.tp = shape, 64, degree
        h, d = shape.hidden, shape.head_dim
        st.dims = {"qkv": (h, shape.qkv_cols // degree), "o": (shape.q_heads * d // degree, h),
                   "gate_up": (h, 2 * shape.intermediate // degree), "down": (shape.intermediate // degree, h)}
        acts = 32 * 2 * 64 * (4096 + 6144 + 4096 + 4096 + 4096 + 28672 + 14336 + 4096)
        assert st.bytes_per_pass() == 3_598_712_832 + acts, degree

"""Tile / Layout / dtype surface: same behaviour as the reference's pyptx.specs / pyptx.types
(pyptx/specs.py:69-209, :363-378; pyptx/types.py:27-105)."""
import pytest

from pyptx_b200 import Layout, Tile, types, unify_envs
from pyptx_b200.types import bf16, f32, from_name


def test_types_surface():
    assert bf16.name == "bf16" and bf16.bits == 16 and bf16.ptx == ".bf16" and repr(f32) == "f32"
    assert from_name(".f32") is f32 and from_name("bf16") is bf16
    assert types.u32 == from_name("u32") and hash(types.u32) == hash(from_name("u32"))
    assert types.pred.bits == 1 and types.b128.bits == 128 and types.e4m3.bits == 8
    with pytest.raises(ValueError, match="Unknown PTX type"):
        from_name("f12")


def test_layout_values():
    assert [l.value for l in Layout] == ["row", "col", "tma_128b", "tma_64b", "tma_32b", "interleaved"]


def test_tile_positional_and_keyword_forms():
    t = Tile("M", "K", bf16, Layout.TMA_128B, tma_box=(128, 64))
    assert t.shape == ("M", "K") and t.dtype is bf16 and t.layout is Layout.TMA_128B
    assert t.tma_box == (128, 64) and t.tma_rank == 2 and t.tma_padding is False
    assert t.rank == 2 and t.symbolic_dims == ("M", "K")
    u = Tile(4, 8, dtype=f32)
    assert u.layout is Layout.ROW and u.shape == (4, 8) and repr(u) == "Tile(4, 8, f32, ROW)"
    assert Tile(4, 8, f32) == u and hash(Tile(4, 8, f32)) == hash(u) and Tile(4, 8, bf16) != u
    with pytest.raises(AttributeError):
        u.shape = (1,)


def test_tile_errors():
    with pytest.raises(ValueError, match="requires a dtype"):
        Tile(4, 8)
    with pytest.raises(ValueError, match="at least one dimension"):
        Tile(f32)
    with pytest.raises(ValueError, match="two dtypes"):
        Tile(4, f32, bf16)
    with pytest.raises(TypeError, match="must be int, str, PtxType, or Layout"):
        Tile(4.5, f32)


def test_resolve_extract_match():
    t = Tile("M", 64, f32)
    assert t.resolve_shape({"M": 12}) == (12, 64)
    with pytest.raises(KeyError, match="not bound"):
        t.resolve_shape({})
    assert t.extract_env((7, 64)) == {"M": 7}
    with pytest.raises(ValueError, match="rank mismatch"):
        t.extract_env((7,))
    with pytest.raises(ValueError, match="dim mismatch: expected 64, got 32"):
        t.extract_env((7, 32))
    assert t.matches((7, 64), "f32") and t.matches((7, 64), "float32")
    assert not t.matches((7, 32), "f32") and not t.matches((7, 64), "bf16") and not t.matches((7,), "f32")
    assert Tile(2, 3, bf16).nbytes() == 12


def test_unify_envs():
    assert unify_envs([{"M": 1, "K": 2}, {"K": 2, "N": 3}]) == {"M": 1, "K": 2, "N": 3}
    with pytest.raises(ValueError, match="conflicting values"):
        unify_envs([{"K": 2}, {"K": 4}])


def test_host_pipeline_rejects_bad_depth_before_touching_cuda():
    from pyptx_b200.host_pipeline import HostPipeline

    with pytest.raises(ValueError, match="depth"):
        HostPipeline(lambda *a: None, depth=0)


def test_reference_entry_points_exist_with_their_signatures():
    """Names and keyword sets of the reference's builders on this path (its example modules), so
    that a caller switching imports finds every one of them."""
    import inspect

    from pyptx_b200.examples.blackwell import gemm_highperf_blackwell as g, grouped_gemm, layer_norm, rms_norm, swiglu
    from pyptx_b200.examples.hopper import softmax
    from pyptx_b200.examples.hopper.experimental import flash_attention_hopper as fa

    want = {
        g.build_gemm: ["M", "N", "K", "arch", "stages", "grid_minor_dim", "grid_tile_width"],
        g.build_gemm_persistent: ["M", "N", "K", "arch", "stages", "grid_minor_dim", "grid_tile_width", "num_ctas"],
        g.build_gemm_2sm: ["M", "N", "K", "arch", "stages", "grid_minor_dim", "grid_tile_width"],
        grouped_gemm.build_grouped_gemm: ["G", "M", "N", "K", "arch"],
        rms_norm.build_rms_norm: ["B", "N", "eps"],
        layer_norm.build_layer_norm: ["B", "N", "eps", "rows_per_cta"],
        swiglu.build_fused_silu_mul: ["M", "F", "rows_per_cta"],
        softmax.build_softmax: ["B", "N", "arch"],
        fa.build_flash_attention_hopper: ["M_q", "N_seq", "head_dim", "sm_scale"],
    }
    for fn, names in want.items():
        params = list(inspect.signature(fn).parameters)
        assert params[:len(names)] == names or all(n in params for n in names), (fn.__name__, params)
    assert inspect.signature(g.build_gemm_persistent).parameters["grid_tile_width"].default == 8
    assert inspect.signature(g.build_gemm_2sm).parameters["stages"].default == 5

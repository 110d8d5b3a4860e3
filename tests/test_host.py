"""CPU: the C-ABI library loads and exports what the header declares; the host-side mirror of
the reference's module behaves like it where no GPU is needed, and fails loudly where one is."""
import ctypes
import os
import re

import pytest
import torch
import torch.nn as nn

from conftest import ROOT, as_half


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "hy3d_int8.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hy3d_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(build_mod):
    lib = build_mod.load_library()
    names = _declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in hy3d_int8.h but not exported"


def test_binding_table_covers_header(build_mod):
    binding = __import__("importlib").import_module("hunyuan3d-tools_b200.csrc._binding")
    declared = set(_declared_symbols())
    bound = set(binding.SIGNATURES) | {"hy3d_arch", "hy3d_status_string",
                                       "hy3d_static_scratch_max_bytes", "hy3d_static_scratch_max_rows",
                                       "hy3d_source_digest", "hy3d_groupnorm_workspace_floats"}
    assert declared == bound


def test_library_identity(build_mod):
    binding = __import__("importlib").import_module("hunyuan3d-tools_b200.csrc._binding")
    lib = binding.configure(build_mod.load_library())
    assert lib.hy3d_arch() == b"sm_100a"
    assert lib.hy3d_version() == binding.ABI_VERSION
    assert lib.hy3d_source_digest().decode() == build_mod._source_digest()
    assert b"alignment" in lib.hy3d_status_string(2)


def test_build_flags_are_sm100a_only(build_mod):
    flags = " ".join(build_mod.cuda_flags())
    assert "arch=compute_100a,code=sm_100a" in flags
    assert "use_fast_math" not in flags
    assert flags.count("-gencode") == 1


def test_loader_names_match_reference(build_mod):
    for name in ("load_int8_kernels", "load_tc_gemm", "load_sparse_tc"):
        assert callable(getattr(build_mod, name))
    tc = build_mod.load_tc_gemm()
    sp = build_mod.load_sparse_tc()
    ik = build_mod.load_int8_kernels()
    for fn in ("int8_linear_tc", "int8_gemm_tc"):
        assert callable(getattr(tc, fn))
    for fn in ("sparse_prune_compress", "sparse_prune_and_pack", "sparse_quantize_act",
               "sparse_int8_gemm", "sparse_int8_linear", "sparse_int8_linear_ex",
               "sparse_int8_linear_path", "test_mma_sp"):
        assert callable(getattr(sp, fn))
    for fn in ("fused_quantize_activation", "fused_dequantize_bias", "int8_linear_fused"):
        assert callable(getattr(ik, fn))


def test_from_linear_matches_reference_buffers(qu, golden):
    lin = nn.Linear(320, 128).half()
    lin.weight.data = as_half(golden["a_weight"])
    lin.bias.data = as_half(golden["a_bias"])
    layer = qu.Int8Linear.from_linear(lin)
    assert torch.equal(layer.weight_int8_nk, torch.from_numpy(golden["a_weight_int8_nk"]))
    assert torch.equal(layer.weight_scale, as_half(golden["a_weight_scale"]))
    assert torch.equal(layer.bias, as_half(golden["a_layer_bias"]))
    assert layer.weight_int8_nk.shape == (128, 320) and layer.weight_int8_nk.dtype == torch.int8
    assert layer.mode == "tc" and layer._tc_ok and layer._sparse_ok
    assert set(dict(layer.named_buffers())) == {"weight_int8_nk", "weight_scale", "bias"}


def test_bf16_source_keeps_bf16_scales(qu):
    lin = nn.Linear(128, 128, bias=False).bfloat16()
    layer = qu.Int8Linear.from_linear(lin)
    assert layer.weight_scale.dtype == torch.bfloat16 and layer.bias is None


def test_model_surgery_stats_match_reference(qu, golden):
    torch.manual_seed(4)
    toy = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 64), nn.Linear(64, 256),
                        nn.Sequential(nn.Linear(256, 256)))
    stats = qu.quantize_model_tensorcore(toy, min_features=128, verbose=False)
    got = [stats["total_params"], stats["quantized_params"], stats["skipped_params"],
           stats["num_replaced"], stats.get("tc_eligible", 0)]
    assert got == golden["toy_stats"].tolist()
    assert isinstance(toy[0], qu.Int8Linear) and isinstance(toy[2], nn.Linear)
    assert isinstance(toy[4][0], qu.Int8Linear)


def test_ineligible_shapes_stay_linear(qu):
    m = nn.Sequential(nn.Linear(200, 256), nn.Linear(256, 136))
    stats = qu.quantize_model_tensorcore(m, verbose=False)
    assert isinstance(m[0], nn.Linear) and isinstance(m[1], nn.Linear)
    assert stats["num_replaced"] == 0 and stats["kept_fp16"] == 2


def test_forward_on_cpu_fails_loudly(qu):
    layer = qu.Int8Linear.from_linear(nn.Linear(128, 128).half())
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(torch.randn(4, 128).half())


def test_sparse_conversion_on_cpu_fails_loudly(qu):
    with pytest.raises(RuntimeError, match="CUDA"):
        qu.Int8Linear.from_linear_sparse(nn.Linear(640, 128).half())


def test_state_dict_roundtrip_dense(qu):
    a = qu.Int8Linear.from_linear(nn.Linear(128, 256).half())
    b = qu.Int8Linear(128, 256, bias=True)
    b.load_state_dict(a.state_dict())
    assert torch.equal(a.weight_int8_nk, b.weight_int8_nk) and torch.equal(a.weight_scale, b.weight_scale)


def test_state_dict_carries_mode_and_epilogue(qu):
    a = qu.Int8Linear.from_linear(nn.Linear(128, 64).bfloat16()).interleave_geglu_rows()
    b = qu.Int8Linear(128, 64, bias=True)
    b.load_state_dict(a.state_dict())
    assert b.epilogue == "geglu" and b.mode == "tc" and b.weight_scale.dtype == torch.bfloat16
    assert torch.equal(a.weight_int8_nk, b.weight_int8_nk) and torch.equal(a.bias, b.bias)


def test_concat_stacks_rows_scales_and_bias(qu):
    torch.manual_seed(3)
    lins = [torch.nn.Linear(128, n, bias=True) for n in (128, 256, 128)]
    layers = [qu.Int8Linear.from_linear(l) for l in lins]
    cat = qu.Int8Linear.concat(layers)
    assert cat.out_features == 512 and cat.in_features == 128 and cat.mode == "tc"
    assert torch.equal(cat.weight_int8_nk, torch.cat([l.weight_int8_nk for l in layers]))
    assert torch.equal(cat.weight_scale, torch.cat([l.weight_scale for l in layers]))
    assert torch.equal(cat.bias, torch.cat([l.bias for l in layers]))
    with pytest.raises(RuntimeError):
        qu.Int8Linear.concat([layers[0], qu.Int8Linear.from_linear(torch.nn.Linear(256, 128))])


def test_qkv_fusion_rewires_attention(qu, pkg):
    import importlib
    un = importlib.import_module(pkg.__name__ + ".unet")
    torch.manual_seed(0)
    blk = un.TransformerBlock(128, 2, 128, 2)
    qu.quantize_model_tensorcore(blk, verbose=False)
    removed = un.fuse_qkv_layers(blk)
    assert removed == 2 + 2 + 1           # two self-attentions (q,k,v -> 1) and one cross-attention (k,v -> 1)
    assert blk.attn1.to_qkv.out_features == 384 and blk.attn1.to_q is None
    assert blk.attn2.to_kv.out_features == 256 and blk.attn2.to_q is not None
    assert un.fuse_qkv_layers(blk) == 0   # idempotent


def test_geglu_row_interleave(qu):
    lin = nn.Linear(128, 64).half()
    layer = qu.Int8Linear.from_linear(lin)
    before = layer.weight_int8_nk.clone()
    layer.interleave_geglu_rows()
    assert layer.epilogue == "geglu"
    assert torch.equal(layer.weight_int8_nk[:16], before[:16])
    assert torch.equal(layer.weight_int8_nk[16:32], before[32:48])
    assert torch.equal(layer.weight_int8_nk[32:48], before[16:32])


def test_oracle_is_not_imported_by_the_product():
    pkg_dir = os.path.join(ROOT, "hunyuan3d-tools_b200")
    for dirpath, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f


def test_build_digest_does_not_depend_on_the_checkout_location(build_mod, tmp_path):
    """A library built here must be accepted as up to date in a copy of the tree elsewhere
    (one process per GPU would otherwise rebuild it concurrently on first use)."""
    import importlib.util
    import shutil
    src_pkg = os.path.join(ROOT, "hunyuan3d-tools_b200", "csrc")
    dst_pkg = tmp_path / "elsewhere" / "hunyuan3d-tools_b200" / "csrc"
    dst_pkg.mkdir(parents=True)
    for name in os.listdir(src_pkg):
        if name.endswith((".cu", ".cuh", ".py")):
            shutil.copy(os.path.join(src_pkg, name), dst_pkg / name)
    shutil.copytree(os.path.join(ROOT, "include"), tmp_path / "elsewhere" / "include")
    spec = importlib.util.spec_from_file_location("build_copy", dst_pkg / "build.py")
    copy = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(copy)
    assert copy._source_digest() == build_mod._source_digest()


def test_state_dict_in_the_reference_buffer_layout_loads(qu):
    """A checkpoint that holds only the reference's buffers (weight_int8_nk, weight_scale,
    bias -- no extra state) loads strictly, also into a layer built without a bias, and a
    sparse one (compressed buffers filled, dense buffer empty) switches the layer to sparse."""
    torch.manual_seed(1)
    src = qu.Int8Linear.from_linear(nn.Linear(128, 64).half())
    sd = {k: v for k, v in src.state_dict().items() if k != "_extra_state"}
    assert set(sd) == {"weight_int8_nk", "weight_scale", "bias"}
    dst = qu.Int8Linear(128, 64, bias=False)
    dst.load_state_dict(sd, strict=True)
    assert dst.mode == "tc" and torch.equal(dst.bias, src.bias)
    assert torch.equal(dst.weight_int8_nk, src.weight_int8_nk)
    sparse_sd = {"weight_int8_nk": torch.empty(0, dtype=torch.int8), "weight_scale": src.weight_scale,
                 "weight_sparse_comp": torch.zeros(64, 64, dtype=torch.int8),
                 "weight_sparse_meta": torch.zeros(64, 4, dtype=torch.int32), "bias": src.bias}
    dst2 = qu.Int8Linear(128, 64)
    dst2.load_state_dict(sparse_sd, strict=True)
    assert dst2.mode == "sparse" and dst2.weight_sparse_comp.shape == (64, 64)


def test_measured_sparse_rule(qu):
    """Mixed assignment by the measured rule: only deep-K layers with many weight rows."""
    assert qu.sparse_pays(1280, 10240) and qu.sparse_pays(5120, 1280)
    for k, n in [(320, 2560), (640, 5120), (1280, 320), (1280, 1280), (2560, 640), (1024, 1280)]:
        assert not qu.sparse_pays(k, n)

"""Host-side checks that need no GPU: the C-ABI library loads and exports every declared symbol, argument
validation rejects bad calls before any launch, and - where the reference source tree is mounted - its modules
really call the dispatch points the way the drop-in functions expect."""
import os
import sys
import types

import pytest
import torch


def test_library_exports_every_declared_symbol(dsb):
    lib = dsb._lib.lib()
    names = dsb._lib.declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), n
        assert n in dsb._lib._SIGS, f"{n} has no ctypes signature"
    assert lib.dsb_version() >= 100


def test_ops_refuse_cpu_tensors(dsb):
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    with pytest.raises(dsb.DsbError):
        dsb.ops.ln_modulate(x, torch.zeros(64), torch.zeros(64))
    with pytest.raises(dsb.DsbError):
        dsb.ops.gemm(x, x)
    with pytest.raises(dsb.DsbError):
        dsb.ops.flash_attn(torch.zeros(1, 4, 1, 128, dtype=torch.bfloat16), torch.zeros(1, 4, 1, 128, dtype=torch.bfloat16),
                           torch.zeros(1, 4, 1, 128, dtype=torch.bfloat16))


def test_synth_is_deterministic():
    synth = __import__("importlib").import_module("diffsynth_engine_b200.synth")
    a = synth.make_state_dict(synth.flux_block_shapes("", 256, 2, "double"), seed=0)
    b = synth.make_state_dict(synth.flux_block_shapes("", 256, 2, "double"), seed=0)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert float(a["attn.norm_q_a.weight"].mean()) > 0.9  # norm weights are 1 + N(0, 0.02)
    n = sum(torch.empty(s, device="meta").numel() for s in synth.flux_dit_shapes().values())
    assert 11.8e9 < n < 12.0e9  # Flux.1-dev has 11.9 G parameters


REF = os.environ.get("DSB_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference"))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "diffsynth_engine")), reason="reference tree not mounted")
def test_reference_modules_use_the_seams():
    """Rebind flux_dit._attn_func / wan_dit.attention / F.linear in the imported reference and check the call
    shapes the drop-in functions are written for."""
    m = types.ModuleType("diffsynth_engine")
    m.__path__ = [os.path.join(REF, "diffsynth_engine")]
    sys.modules.setdefault("diffsynth_engine", m)
    from diffsynth_engine.models.flux import flux_dit
    from diffsynth_engine.models.wan import wan_dit
    from diffsynth_engine.models.basic.transformer_helper import RoPEEmbedding
    import torch.nn.functional as F
    seen = {}

    def fake_attn(q, k, v):
        seen["flux"] = (tuple(q.shape), q.stride(-1), tuple(v.shape), v.is_contiguous(), v.stride(-1))
        return F.scaled_dot_product_attention(q, k, v)

    d, H = 256, 2
    blk = flux_dit.FluxSingleTransformerBlock(d, H, device="cpu", dtype=torch.float32)
    ids = torch.zeros(1, 12, 3)
    rope = RoPEEmbedding(d, 10000, [16, 56, 56])(ids)
    old = flux_dit._attn_func
    flux_dit._attn_func = fake_attn
    try:
        blk(torch.randn(1, 12, d), None, torch.randn(1, d), rope)
    finally:
        flux_dit._attn_func = old
    shape_q, q_inner, shape_v, v_contig, v_inner = seen["flux"]
    assert shape_q == (1, H, 12, 128) and q_inner == 1      # [B,H,S,D] (strides follow the fused projection)
    assert shape_v == (1, H, 12, 128) and not v_contig and v_inner == 1   # strided view of the fused projection

    def fake_wan_attention(q, k, v, num_heads):
        seen["wan"] = (tuple(q.shape), tuple(k.shape), num_heads)
        return torch.zeros_like(q)

    sa = wan_dit.CrossAttention(d, H, device="cpu", dtype=torch.float32)
    old = wan_dit.attention
    wan_dit.attention = fake_wan_attention
    try:
        sa(torch.randn(1, 9, d), torch.randn(1, 5, d))
    finally:
        wan_dit.attention = old
    assert seen["wan"] == ((1, 9, d), (1, 5, d), H)       # [B,S,H*D] in, looked up at call time

    calls = []
    origin = F.linear

    def spy(x, w, b=None):
        calls.append((tuple(x.shape), tuple(w.shape)))
        return origin(x, w, b)

    F.linear = spy
    try:
        torch.nn.Linear(8, 4)(torch.randn(2, 3, 8))
    finally:
        F.linear = origin
    assert calls == [((2, 3, 8), (4, 8))]                 # nn.Linear resolves F.linear at call time, [N,K] weight


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "diffsynth_engine")), reason="reference tree not mounted")
def test_reference_lora_linear_has_what_the_fused_path_reads(dsb):
    """The fused-LoRA seam reads ``_lora_dict`` adapters (scale, alpha, rank, up.weight, down.weight) off the
    reference's LoRALinear and swaps its forward; check that against the real class, on the CPU."""
    m = types.ModuleType("diffsynth_engine")
    m.__path__ = [os.path.join(REF, "diffsynth_engine")]
    saved = sys.modules.get("diffsynth_engine")
    sys.modules["diffsynth_engine"] = m
    try:
        from diffsynth_engine.models.basic.lora import LoRALinear
        lora = __import__("importlib").import_module("diffsynth_engine_b200.lora")
        lin = LoRALinear(32, 16)
        lin.add_lora("a", 0.5, 4, 8, torch.randn(16, 4), torch.randn(4, 32), "cpu", torch.float32)
        (coef, up, down), = lora._adapters(lin)
        assert coef == 0.5 * 8 / 4 and up.shape == (16, 4) and down.shape == (4, 32)
        sig = lora._signature(lin)
        lin.modify_scale("a", 0.25)
        assert lora._signature(lin) != sig                      # a scale change invalidates the built extension
        assert lora.fuse_lora(lin) == 0                         # not prepacked: left alone
    finally:
        if saved is None:
            sys.modules.pop("diffsynth_engine", None)
        else:
            sys.modules["diffsynth_engine"] = saved


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "diffsynth_engine")), reason="reference tree not mounted")
def test_reference_gguf_parameter_is_recognised(dsb):
    """``enable_b200_linear`` finds Q8_0 weights by the ``quant_dtype`` tag of the reference's GGUFParameter and reads
    their stored bytes, not the dequantised ``shape``/``dtype`` the class reports."""
    import gguf
    m = types.ModuleType("diffsynth_engine")
    m.__path__ = [os.path.join(REF, "diffsynth_engine")]
    saved = sys.modules.get("diffsynth_engine")
    sys.modules["diffsynth_engine"] = m
    try:
        from diffsynth_engine.utils.gguf import GGUFParameter
        quant = __import__("importlib").import_module("diffsynth_engine_b200.quant")
        raw = torch.zeros(8, 2 * 34, dtype=torch.uint8)
        p = GGUFParameter(raw, quant_dtype=gguf.GGMLQuantizationType.Q8_0, compute_dtype=torch.bfloat16)
        assert tuple(p.shape) == (8, 64) and p.dtype == torch.bfloat16      # what the class reports
        assert quant._is_gguf_q8_0(p)
        assert tuple(quant._raw_bytes(p).shape) == (8, 68) and quant._raw_bytes(p).dtype == torch.uint8
        q4 = GGUFParameter(torch.zeros(8, 144, dtype=torch.uint8), quant_dtype=gguf.GGMLQuantizationType.Q4_K,
                           compute_dtype=torch.bfloat16)
        assert not quant._is_gguf_q8_0(q4) and quant._gguf_type(q4) == "Q4_K"
        q6 = GGUFParameter(raw, quant_dtype=gguf.GGMLQuantizationType.Q6_K, compute_dtype=torch.bfloat16)
        assert quant._gguf_type(q6) == "Q6_K"                                 # every block format of the reference
        f16 = GGUFParameter(raw, quant_dtype=gguf.GGMLQuantizationType.F16, compute_dtype=torch.bfloat16)
        assert quant._gguf_type(f16) is None                                  # plain tensors stay with the reference
        assert not quant._is_gguf_q8_0(torch.nn.Parameter(torch.zeros(2, 2)))
    finally:
        if saved is None:
            sys.modules.pop("diffsynth_engine", None)
        else:
            sys.modules["diffsynth_engine"] = saved


def test_entry_points_reject_bad_arguments_without_a_gpu(dsb):
    """Every entry point validates its arguments before it touches CUDA and answers with DSB_ERR_ARG (-1) or
    DSB_ERR_UNSUPPORTED (-4); none of these calls launches anything, so they run on a machine without a GPU."""
    import ctypes
    lib = dsb._lib.lib()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) // 16 * 16
    # Q8_0: K must be a multiple of 32, rows 2-byte aligned and long enough
    assert lib.dsb_dequant_q8_0(p16, 68, 4, 48, p16, 64, None) == -1
    assert lib.dsb_dequant_q8_0(p16, 33, 4, 64, p16, 64, None) == -1
    assert lib.dsb_dequant_q8_0(p16, 34, 4, 64, p16, 64, None) == -1          # 64 weights need 68 bytes per row
    assert lib.dsb_dequant_q8_0(None, 68, 0, 64, None, 64, None) == 0         # no rows: nothing to do
    # Q4_K: K a multiple of 256, 16-byte aligned rows of 144-byte super-blocks
    assert lib.dsb_dequant_q4_k(p16, 144, 2, 128, p16, 128, None) == -1
    assert lib.dsb_dequant_q4_k(p16 + 8, 144, 2, 256, p16, 256, None) == -1
    assert lib.dsb_dequant_q4_k(p16, 100, 2, 256, p16, 256, None) == -1
    # cast: split form only for e4m3; widths in multiples of 8
    assert lib.dsb_cast_quant(p16, 64, p16, 64, 4, 64, 2, 1, None) == -1
    assert lib.dsb_cast_quant(p16, 64, p16, 64, 4, 60, 1, 0, None) == -1
    # attention: head_dim 128 only, strides in multiples of 8 elements
    st = [128 * 4, 128, 128 * 4 * 0 + 128] * 4
    assert lib.dsb_flash_attn(p16, p16, p16, p16, 1, 1, 4, 4, 64, *st, 1.0, None, None) == -4
    bad = list(st)
    bad[1] = 12
    assert lib.dsb_flash_attn(p16, p16, p16, p16, 1, 1, 4, 4, 128, *bad, 1.0, None, None) == -1
    # GEMM group: 1 or 2 problems; e4m3 output cannot be combined with the residual form or a misaligned pitch
    g = (dsb._lib.GemmArgs * 1)()
    a = g[0]
    a.A, a.lda, a.W, a.ldw, a.M, a.N, a.K = p16, 64, p16, 64, 8, 64, 64
    a.out0, a.ld_out0, a.split_col = p16, 64, 64
    assert lib.dsb_gemm_group(g, 3, 1, None, None) == -1
    a.out0_fmt, a.resid, a.ld_resid = 1, p16, 64
    assert lib.dsb_gemm_group(g, 1, 1, None, None) == -1
    a.resid, a.ld_resid, a.ld_out0 = None, 0, 72
    assert lib.dsb_gemm_group(g, 1, 1, None, None) == -1
    a.out0_fmt, a.ld_out0, a.N = 0, 64, 60                                     # N must be a multiple of 8
    assert lib.dsb_gemm_group(g, 1, 1, None, None) == -1


def test_new_entry_points_reject_bad_arguments_without_a_gpu(dsb):
    """The entry points added for the sequence-parallel attention, the boundary kernels and the GGUF formats check
    their arguments before touching CUDA."""
    import ctypes
    lib = dsb._lib.lib()
    buf = (ctypes.c_char * 4096)()
    p16 = (ctypes.addressof(buf) + 15) // 16 * 16
    one = (ctypes.c_void_p * 1)(p16)
    two = (ctypes.c_void_p * 2)(p16, p16)
    none2 = (ctypes.c_void_p * 2)(p16, None)
    st = [512, 128] * 4                                                        # (token, head) strides of q, k, v, o
    # attention over parts: 1..8 parts that cover Sq, query parts in whole 128-row tiles, no null part
    assert lib.dsb_flash_attn_parts(two, 2, 100, p16, p16, two, 2, 128, 4, 256, 256, 128, *st, 1.0, None, 0, None, None) == -1
    assert lib.dsb_flash_attn_parts(two, 2, 128, p16, p16, two, 2, 64, 4, 256, 256, 128, *st, 1.0, None, 0, None, None) == -1
    assert lib.dsb_flash_attn_parts(two, 9, 128, p16, p16, two, 2, 128, 4, 256, 256, 128, *st, 1.0, None, 0, None, None) == -1
    assert lib.dsb_flash_attn_parts(none2, 2, 128, p16, p16, two, 2, 128, 4, 256, 256, 128, *st, 1.0, None, 0, None, None) == -1
    assert lib.dsb_flash_attn_parts(two, 2, 128, p16, p16, two, 2, 128, 4, 256, 256, 64, *st, 1.0, None, 0, None, None) == -4
    assert lib.dsb_flash_attn_parts(two, 2, 128, p16, p16, two, 2, 128, 4, 256, 256, 128, *st, 1.0, p16 + 4, 64, None, None) == -1
    # e4m3 attention output: strides in multiples of 16 bytes
    s12 = [2048, 512, 128] * 3 + [2048, 520, 128]
    assert lib.dsb_flash_attn_out8(p16, p16, p16, p16, 1, 4, 4, 4, 128, *s12, 1.0, None, None) == -1
    # rank barrier: 1..8 ranks, own rank inside the group, aligned flag arrays, a positive wait limit
    assert lib.dsb_rank_barrier(one, 0, 0, 1, 1000, None, None) == -1
    assert lib.dsb_rank_barrier(two, 2, 2, 1, 1000, None, None) == -1
    assert lib.dsb_rank_barrier(none2, 2, 0, 1, 1000, None, None) == -1
    assert lib.dsb_rank_barrier(one, 1, 0, 1, 0, None, None) == -1
    # patchify / unpatchify: at most 128 channels, rows at least C*4 wide, 8-bit formats need the scale array
    assert lib.dsb_patchify(p16, 200, 1, 2, 2, 0, 4, 0, p16, 800, None, None) == -1
    assert lib.dsb_patchify(p16, 16, 1, 2, 2, 0, 4, 0, p16, 32, None, None) == -1
    assert lib.dsb_patchify(p16, 16, 1, 2, 2, 0, 4, 1, p16, 64, None, None) == -1
    assert lib.dsb_patchify(p16, 16, 1, 2, 2, 0, 0, 0, None, 64, None, None) == 0     # no rows: nothing to do
    assert lib.dsb_unpatchify(p16, 32, 16, 1, 2, 2, 1, p16, None) == -1
    # GGUF: unknown block type, K not a multiple of the block size
    assert lib.dsb_dequant_gguf(99, p16, 144, 2, 256, p16, 256, None) == -4            # DSB_ERR_UNSUPPORTED
    assert lib.dsb_dequant_gguf(14, p16, 210, 2, 200, p16, 200, None) == -1
    assert int(lib.dsb_flash_attn_workspace_bytes()) >= 0 or True                      # needs a device; only that it links


def test_gemm_front_end_checks_shapes_and_dtypes_before_any_launch(dsb):
    """``ops._check_gemm_io`` is what stands between a tensor and a raw pointer: it accepts what the engines pass
    (row slices, wider pitches, one-element scales) and rejects what the kernel would overrun."""
    import torch
    chk = dsb.ops._check_gemm_io
    M, N = 64, 128
    bf, f32, e4 = torch.bfloat16, torch.float32, torch.float8_e4m3fn
    out = torch.zeros(M, N, dtype=bf)
    wide = torch.zeros(M, 3 * N, dtype=bf)
    chk(M, N, out, None, None)
    chk(M, N, wide[:, N:2 * N], None, None, resid=wide[:, :N], row_scale=torch.zeros(M), col_scale=torch.zeros(1),
        bias=torch.zeros(N), gate=torch.zeros(N))
    chk(M, N, torch.zeros(M, 32, dtype=bf), torch.zeros(M, 96, dtype=e4), 32, e4m3_ok=True)
    for bad in (dict(out=torch.zeros(M, N - 8, dtype=bf)), dict(out=torch.zeros(M + 1, N, dtype=bf)),
                dict(out=torch.zeros(M, N, dtype=torch.float16)), dict(out=torch.zeros(M, N, dtype=e4)),
                dict(out=out.t().contiguous().t()), dict(out=out, resid=torch.zeros(M, N, dtype=f32)),
                dict(out=out, resid=torch.zeros(M, N - 8, dtype=bf)), dict(out=out, row_scale=torch.zeros(M - 1)),
                dict(out=out, bias=torch.zeros(N, dtype=bf)), dict(out=out, gate=torch.zeros(N - 1)),
                dict(out=out, col_scale=torch.zeros(N // 2))):
        with pytest.raises(dsb.DsbError):
            chk(M, N, bad["out"], None, None, bad.get("resid"), bad.get("row_scale"), bad.get("col_scale"),
                bad.get("bias"), bad.get("gate"))
    with pytest.raises(dsb.DsbError):                                   # a split needs 0 < split_col < N
        chk(M, N, torch.zeros(M, N, dtype=bf), torch.zeros(M, N, dtype=bf), N, e4m3_ok=True)

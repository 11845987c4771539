"""GPU parity of ttb_matmul against an fp32 torch matmul of the oracle-unpacked weights.

Tolerances (from the task statement, written out): PCC >= 0.9999 with the reference's comp_pcc definition, and
max|y - y_ref| / max|y_ref| <= 1e-2."""
import numpy as np
import pytest

import cabi
import oracle
import vectors

pytestmark = pytest.mark.gpu
PCC_MIN = 0.9999
MAX_REL = 1e-2


def make_case(ttb, orc, seed, M, K, N, w_dtype, w_std=0.02):
    import torch
    x = vectors.randn(seed, (M, K), 1.0).bfloat16()
    w = vectors.randn(seed + 1000, (K, N), w_std)
    if w_dtype == cabi.BFLOAT16:
        wq = w.bfloat16()
        w_dev = ttb.tilize(wq.cuda(), 1, K, N)
        w_ref = wq.float()
    else:
        ofmt = 0 if w_dtype == cabi.BFLOAT8_B else 1
        packed = orc.from_torch(w.numpy(), ofmt, 1, K, N)          # weights packed by the ORACLE, not the GPU
        w_dev = torch.from_numpy(packed).cuda()
        w_ref = torch.from_numpy(orc.to_torch(packed, ofmt, 1, K, N).reshape(K, N).copy())
    return x, w_dev, w_ref


def check(y, y_ref):
    y, y_ref = y.float().cpu().numpy(), y_ref.float().cpu().numpy()
    pcc = oracle.comp_pcc(y_ref, y)
    rel = np.abs(y - y_ref).max() / np.abs(y_ref).max()
    assert pcc >= PCC_MIN, f"PCC {pcc}"
    assert rel <= MAX_REL, f"max relative error {rel}"


def act_ref(y, act):
    import torch
    if act == cabi.ACT_RELU:
        return torch.relu(y)
    if act == cabi.ACT_GELU:
        return torch.nn.functional.gelu(y)
    if act == cabi.ACT_SILU:
        return torch.nn.functional.silu(y)
    return y


SHAPES_SMALL = [(32, 64, 128), (32, 128, 128), (32, 64, 256), (32, 512, 384), (64, 256, 256), (128, 192, 128), (96, 128, 128),
                (32, 32, 32), (64, 96, 160)]


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B, cabi.BFLOAT16])
@pytest.mark.parametrize("M,K,N", SHAPES_SMALL)
@pytest.mark.parametrize("generic", [False, True])
def test_matmul_small_shapes(ttb, orc, w_dtype, M, K, N, generic):
    import torch
    x, w_dev, w_ref = make_case(ttb, orc, 5, M, K, N, w_dtype)
    a = ttb.tilize(x.cuda(), 1, M, K)
    flags = cabi.MM_FORCE_GENERIC if generic else 0
    y = ttb.untilize(ttb.matmul(a, w_dev, w_dtype, 1, M, K, N, flags=flags), 1, M, N).reshape(M, N)
    y_ref = x.float() @ w_ref
    check(y, y_ref)


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
def test_tensor_core_kernel_agrees_with_generic_kernel(ttb, orc, w_dtype):
    """Same operands, fp32 accumulation in both: results may differ only by summation order."""
    import torch
    M, K, N = 32, 1024, 512
    x, w_dev, _ = make_case(ttb, orc, 9, M, K, N, w_dtype)
    a = ttb.tilize(x.cuda(), 1, M, K)
    y1 = ttb.matmul(a, w_dev, w_dtype, 1, M, K, N, out_fp32=True)
    y2 = ttb.matmul(a, w_dev, w_dtype, 1, M, K, N, out_fp32=True, flags=cabi.MM_FORCE_GENERIC)
    assert torch.allclose(y1, y2, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("act", [cabi.ACT_NONE, cabi.ACT_RELU, cabi.ACT_GELU, cabi.ACT_SILU])
@pytest.mark.parametrize("generic", [False, True])
def test_linear_bias_activation_and_layout_flags(ttb, orc, act, generic):
    import torch
    M, K, N = 32, 256, 384
    x, w_dev, w_ref = make_case(ttb, orc, 21, M, K, N, cabi.BFLOAT8_B)
    bias = vectors.randn(77, (N,), 0.5).bfloat16()
    bias_tile = torch.zeros(32, N, dtype=torch.bfloat16)
    bias_tile[0] = bias
    b_dev = ttb.tilize(bias_tile.cuda(), 1, 32, N)
    y_ref = act_ref(x.float() @ w_ref + bias.float(), act)
    base = cabi.MM_FORCE_GENERIC if generic else 0
    # tiled in, tiled out
    a = ttb.tilize(x.cuda(), 1, M, K)
    y = ttb.untilize(ttb.matmul(a, w_dev, cabi.BFLOAT8_B, 1, M, K, N, bias=b_dev, act=act, flags=base), 1, M, N).reshape(M, N)
    check(y, y_ref)
    # row-major in, row-major out, fp32 out
    y2 = ttb.matmul(x.cuda().contiguous(), w_dev, cabi.BFLOAT8_B, 1, M, K, N, bias=b_dev, act=act,
                    flags=base | cabi.MM_A_ROW_MAJOR | cabi.MM_OUT_ROW_MAJOR, out_fp32=True).reshape(M, N)
    check(y2, y_ref)


@pytest.mark.parametrize("M,K,N,w_dtype,seed", [
    (32, 4544, 18176, cabi.BFLOAT8_B, 1),      # Falcon-7B h_to_4h decode
    (32, 4096, 4096, cabi.BFLOAT8_B, 2),       # Mistral Wq / Wo (K split over blocks)
    (32, 4096, 1024, cabi.BFLOAT8_B, 2),       # Mistral Wk / Wv
    (32, 4096, 14336, cabi.BFLOAT4_B, 2),      # Mistral w1 / w3
    (32, 14336, 4096, cabi.BFLOAT8_B, 2),      # Mistral w2
    (32, 8192, 3584, cabi.BFLOAT8_B, 4),       # Llama-70B w1 shard at 8 GPUs
])
def test_decode_shapes_of_the_benchmark_configurations(ttb, orc, M, K, N, w_dtype, seed):
    import torch
    x, w_dev, w_ref = make_case(ttb, orc, seed, M, K, N, w_dtype)
    a = ttb.tilize(x.cuda(), 1, M, K)
    y = ttb.untilize(ttb.matmul(a, w_dev, w_dtype, 1, M, K, N), 1, M, N).reshape(M, N)
    y_ref = (x.float().cuda() @ w_ref.cuda())
    check(y, y_ref)


def make_big_case(ttb, orc, seed, K, N, w_dtype, slice_cols=1024):
    """A weight too large for the host oracle to pack whole in test time: generated and packed on the GPU, with a seeded
    slice of `slice_cols` columns also packed and unpacked by the ORACLE and compared byte for byte with the same tiles
    of the GPU result (the conversion tests pin the packer everywhere else). Returns the packed weight and the fp32
    matrix of its unpacked values, both on the device."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(K, N, generator=g, device="cuda") * 0.02
    packed = ttb.pack(w, w_dtype, 1, K, N)
    w_ref = ttb.unpack(packed, w_dtype, 1, K, N).reshape(K, N)
    cols = min(slice_cols, N)
    c0 = ((seed * 7919) % (N - cols + 32)) // 32 * 32 if N > cols else 0
    ofmt = 0 if w_dtype == cabi.BFLOAT8_B else 1
    tb = cabi.TILE_BYTES[w_dtype]
    want = orc.from_torch(w[:, c0:c0 + cols].contiguous().cpu().numpy(), ofmt, 1, K, cols)
    got = packed.reshape(K // 32, N // 32, tb)[:, c0 // 32:(c0 + cols) // 32].contiguous().cpu().numpy().reshape(-1)
    assert np.array_equal(got, want), "GPU-packed tiles differ from the oracle's on the checked column slice"
    want_f = orc.to_torch(want, ofmt, 1, K, cols).reshape(K, cols)
    assert np.array_equal(w_ref[:, c0:c0 + cols].cpu().numpy(), want_f), "GPU-unpacked values differ from the oracle's"
    del w
    return packed, w_ref


# Llama-2-70B decode, the configuration the benchmark times: per layer and per GPU (G = 1, 2, 4, 8 column shards) one
# launch for q/k/v, one for wo, one for w1/w3 and one for w2; batch 32, seed 4.
LLAMA_SINGLE = [(8192, 8192 // G) for G in (1, 2, 4, 8)] + [(28672, 8192 // G) for G in (1, 2, 4, 8)]
LLAMA_GROUPS = [(8192, [8192 // G, 1024 // G, 1024 // G]) for G in (1, 2, 4, 8)] + [(8192, [28672 // G, 28672 // G]) for G in (1, 2, 4, 8)]


@pytest.mark.parametrize("K,N", LLAMA_SINGLE)
def test_llama70b_decode_single_weight_launches(ttb, orc, K, N):
    import torch
    M = 32
    packed, w_ref = make_big_case(ttb, orc, 4 + N, K, N, cabi.BFLOAT8_B)
    x = vectors.randn(4, (M, K), 1.0).bfloat16()
    a = ttb.tilize(x.cuda(), 1, M, K)
    y = ttb.untilize(ttb.matmul(a, packed, cabi.BFLOAT8_B, 1, M, K, N), 1, M, N).reshape(M, N)
    check(y, x.float().cuda() @ w_ref)


@pytest.mark.parametrize("K,Ns", LLAMA_GROUPS)
def test_llama70b_decode_grouped_launches(ttb, orc, K, Ns):
    """The q/k/v and w1/w3 launches of the timed step (ttb_matmul_multi), every output against the fp32 reference."""
    import ctypes
    import torch
    M = 32
    x = vectors.randn(4, (M, K), 1.0).bfloat16()
    a = ttb.tilize(x.cuda(), 1, M, K)
    cases = [make_big_case(ttb, orc, 4 + 13 * j + N, K, N, cabi.BFLOAT8_B) for j, N in enumerate(Ns)]
    outs = [torch.empty(M * N, dtype=torch.bfloat16, device="cuda") for N in Ns]
    n = len(Ns)
    arr_w = (ctypes.c_void_p * n)(*[c[0].data_ptr() for c in cases])
    arr_o = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
    arr_n = (ctypes.c_int64 * n)(*Ns)
    nbytes = ttb.matmul_multi_workspace_bytes(cabi.BFLOAT8_B, 1, M, K, n, arr_n)
    ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    for rep in range(2):
        ttb.check(ttb.cdll.ttb_matmul_multi(a.data_ptr(), cabi.BFLOAT16, n, arr_w, cabi.BFLOAT8_B, None, arr_o, cabi.BFLOAT16, 1, M, K, arr_n,
                                            cabi.ACT_NONE, cabi.MM_WORKSPACE_ZEROED | cabi.MM_WEIGHTS_RESIDENT, ws.data_ptr(), nbytes, None, None, None))
        ttb.check(ttb.check_status(None))
        for j, N in enumerate(Ns):
            check(ttb.untilize(outs[j], 1, M, N).reshape(M, N), x.float().cuda() @ cases[j][1])


@pytest.mark.parametrize("M,K,N", [(32, 64, 128), (32, 96, 128), (32, 416, 256), (64, 256, 256), (128, 192, 128), (32, 4544, 18176), (32, 4096, 1024),
                                   (256, 1024, 512), (64, 4096, 2048), (128, 8192, 1024), (96, 2048, 640)])
def test_both_decode_kernels_agree_with_the_generic_kernel(ttb, orc, M, K, N):
    """bfloat8_b decode shapes run on the kernel that feeds weights to the MMA through tensor memory (default) or on the
    one that expands them into shared memory (MM_DECODE_SMEM_OPERAND): same operands, fp32 accumulation, so both must
    agree with the CUDA-core kernel up to summation order, including rows with exponents above 127."""
    import torch
    x, w_dev, w_ref = make_case(ttb, orc, 17, M, K, N, cabi.BFLOAT8_B, w_std=0.02 if K != 96 else 3.0)
    a = ttb.tilize(x.cuda(), 1, M, K)
    y2 = ttb.matmul(a, w_dev, cabi.BFLOAT8_B, 1, M, K, N, out_fp32=True, flags=cabi.MM_FORCE_GENERIC)
    scale = y2.abs().max().item()
    for flags in (0, cabi.MM_DECODE_SMEM_OPERAND):
        y1 = ttb.matmul(a, w_dev, cabi.BFLOAT8_B, 1, M, K, N, out_fp32=True, flags=flags)
        assert torch.allclose(y1, y2, rtol=1e-4, atol=1e-4 * scale)
        check(ttb.untilize(y1, 1, M, N).reshape(M, N), x.float().cuda() @ w_ref.cuda())


def test_weights_with_large_magnitudes(ttb, orc):
    """Rows whose shared exponent exceeds 127 (values of 2 and above) take the second-multiply path of the expanders."""
    import torch
    M, K, N = 32, 256, 256
    for w_dtype in (cabi.BFLOAT8_B, cabi.BFLOAT4_B):
        x, w_dev, w_ref = make_case(ttb, orc, 23, M, K, N, w_dtype, w_std=40.0)
        a = ttb.tilize(x.cuda(), 1, M, K)
        y = ttb.untilize(ttb.matmul(a, w_dev, w_dtype, 1, M, K, N, out_fp32=True), 1, M, N).reshape(M, N)
        check(y, x.float() @ w_ref)


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
@pytest.mark.parametrize("M,K,N", [(512, 64, 128), (512, 256, 256), (640, 96, 128), (1024, 160, 384), (2048, 512, 256),
                                   (512, 64, 19200)])   # the last one: 150 blocks = one wave + a tail launch of small blocks
def test_prefill_kernel_small_shapes(ttb, orc, w_dtype, M, K, N):
    """Row counts of 512 and more take the compute-bound tensor-core kernel (one or two 128-row accumulators per block)."""
    import torch
    x, w_dev, w_ref = make_case(ttb, orc, 41, M, K, N, w_dtype)
    a = ttb.tilize(x.cuda(), 1, M, K)
    y = ttb.matmul(a, w_dev, w_dtype, 1, M, K, N, out_fp32=True)
    y2 = ttb.matmul(a, w_dev, w_dtype, 1, M, K, N, out_fp32=True, flags=cabi.MM_FORCE_GENERIC)
    assert torch.allclose(y, y2, rtol=1e-4, atol=1e-4 * y2.abs().max().item())
    check(ttb.untilize(y, 1, M, N).reshape(M, N), x.float() @ w_ref)


@pytest.mark.parametrize("act", [cabi.ACT_NONE, cabi.ACT_GELU])
def test_prefill_kernel_bias_activation_layouts(ttb, orc, act):
    import torch
    M, K, N = 512, 128, 256
    x, w_dev, w_ref = make_case(ttb, orc, 43, M, K, N, cabi.BFLOAT8_B)
    bias = vectors.randn(78, (N,), 0.5).bfloat16()
    bias_tile = torch.zeros(32, N, dtype=torch.bfloat16)
    bias_tile[0] = bias
    b_dev = ttb.tilize(bias_tile.cuda(), 1, 32, N)
    y_ref = act_ref(x.float() @ w_ref + bias.float(), act)
    a = ttb.tilize(x.cuda(), 1, M, K)
    y = ttb.untilize(ttb.matmul(a, w_dev, cabi.BFLOAT8_B, 1, M, K, N, bias=b_dev, act=act), 1, M, N).reshape(M, N)
    check(y, y_ref)
    y2 = ttb.matmul(x.cuda().contiguous(), w_dev, cabi.BFLOAT8_B, 1, M, K, N, bias=b_dev, act=act,
                    flags=cabi.MM_A_ROW_MAJOR | cabi.MM_OUT_ROW_MAJOR).reshape(M, N)
    check(y2, y_ref)
    # batch of four 128-row slabs sharing the weight
    xb = x.reshape(4, 128, K)
    ab = ttb.tilize(xb.cuda(), 4, 128, K)
    yb = ttb.untilize(ttb.matmul(ab, w_dev, cabi.BFLOAT8_B, 4, 128, K, N, bias=b_dev, act=act), 4, 128, N).reshape(M, N)
    check(yb, y_ref)


def test_prefill_llama70b_mlp_shape(ttb):
    """The compute-bound benchmark configuration at full size: [2048, 8192] x bfloat8_b [8192, 28672], seed 3. The weight is
    packed and unpacked by the GPU kernels (bit-exact with the oracle per the conversion tests); the fp32 golden runs on the GPU."""
    import torch
    M, K, N = 2048, 8192, 28672
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(M, K, generator=g, device="cuda").bfloat16()
    w = torch.randn(K, N, generator=g, device="cuda") * 0.02
    packed = ttb.pack(w, cabi.BFLOAT8_B, 1, K, N)
    w_ref = ttb.unpack(packed, cabi.BFLOAT8_B, 1, K, N).reshape(K, N)
    del w
    a = ttb.tilize(x, 1, M, K)
    y = ttb.untilize(ttb.matmul(a, packed, cabi.BFLOAT8_B, 1, M, K, N), 1, M, N).reshape(M, N).float()
    torch.backends.cuda.matmul.allow_tf32 = False
    y_ref = x.float() @ w_ref
    rel = ((y - y_ref).abs().max() / y_ref.abs().max()).item()
    sample = torch.randint(0, M * N, (2_000_000,), device="cuda")
    pcc = oracle.comp_pcc(y_ref.reshape(-1)[sample].cpu().numpy(), y.reshape(-1)[sample].cpu().numpy())
    assert rel <= MAX_REL and pcc >= PCC_MIN, (rel, pcc)


def test_batched_activations_share_the_weight(ttb, orc):
    import torch
    B, M, K, N = 2, 32, 128, 256
    x = vectors.randn(3, (B, M, K), 1.0).bfloat16()
    _, w_dev, w_ref = make_case(ttb, orc, 3, M, K, N, cabi.BFLOAT8_B)
    a = ttb.tilize(x.cuda(), B, M, K)
    y = ttb.untilize(ttb.matmul(a, w_dev, cabi.BFLOAT8_B, B, M, K, N), B, M, N).reshape(B, M, N)
    check(y, x.float() @ w_ref)


@pytest.mark.parametrize("flags", [cabi.MM_DETERMINISTIC, 0, cabi.MM_DECODE_SMEM_OPERAND, cabi.MM_DECODE_SMEM_OPERAND | cabi.MM_DETERMINISTIC])
def test_repeated_launches_reuse_scratch(ttb, orc, flags):
    """Split-K scratch (arrival counters, accumulation tiles) must be back to zero after each launch. With
    MM_DETERMINISTIC the partial sums are added in a fixed order and repeated launches agree bit for bit; the default
    adds them in arrival order, so repeats may differ in the last fp32 bit before rounding to bf16."""
    import torch
    M, K, N = 32, 4096, 1024
    x, w_dev, w_ref = make_case(ttb, orc, 31, M, K, N, cabi.BFLOAT8_B)
    a = ttb.tilize(x.cuda(), 1, M, K)
    nbytes = ttb.matmul_workspace_bytes(cabi.BFLOAT8_B, 1, M, K, N, 0)
    assert nbytes > 0
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    outs = []
    for _ in range(3):
        out = torch.empty(M * N, dtype=torch.bfloat16, device="cuda")
        ttb.check(ttb.cdll.ttb_matmul(a.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), cabi.BFLOAT8_B, None, out.data_ptr(),
                                      cabi.BFLOAT16, 1, M, K, N, 0, flags | cabi.MM_WORKSPACE_ZEROED, ws.data_ptr(), nbytes, None))
        outs.append(out)
    ttb.check(ttb.check_status(None))
    if flags & cabi.MM_DETERMINISTIC:
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    else:
        assert torch.allclose(outs[0].float(), outs[1].float(), rtol=1e-2, atol=1e-2) and torch.allclose(outs[1].float(), outs[2].float(), rtol=1e-2, atol=1e-2)
    # everything the kernels must leave zero is zero again
    assert int(ws[: 65536 + (16 << 20)].count_nonzero().item()) == 0
    check(ttb.untilize(outs[0], 1, M, N).reshape(M, N), x.float() @ w_ref)
    # too small a workspace is refused before anything is launched
    rc = ttb.cdll.ttb_matmul(a.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), cabi.BFLOAT8_B, None, outs[0].data_ptr(),
                             cabi.BFLOAT16, 1, M, K, N, 0, 0, ws.data_ptr(), 16, None)
    assert rc == -4


@pytest.mark.parametrize("tmem", [0, cabi.MM_DECODE_SMEM_OPERAND])
@pytest.mark.parametrize("M", [32, 128])
def test_overlapped_launches_keep_their_dependencies(ttb, orc, tmem, M):
    """MM_WEIGHTS_RESIDENT lets a decode kernel start while the previous one drains. A chain in which every launch consumes
    the previous launch's output (and all share one workspace) must give exactly the results of the same chain launched
    without overlap; MM_DETERMINISTIC makes both chains bit-reproducible."""
    import torch
    K = N = 4096      # (a shape whose K range is shared out among blocks under every plan: the launches share scratch)
    depth = 6
    x = vectors.randn(77, (M, K), 1.0).bfloat16()
    ws_list = []
    for i in range(depth):
        _, w_dev, _ = make_case(ttb, orc, 80 + i, M, K, N, cabi.BFLOAT8_B, w_std=0.02)
        ws_list.append(w_dev)
    torch.cuda.synchronize()
    nbytes = ttb.matmul_workspace_bytes(cabi.BFLOAT8_B, 1, M, K, N, cabi.MM_DETERMINISTIC | tmem)
    assert nbytes > 0 or (M == 128 and not tmem)      # (two tile rows per block: this shape needs no sharing of K)
    ws = torch.zeros(max(nbytes, 65536), dtype=torch.uint8, device="cuda")

    def chain(extra):
        cur = ttb.tilize(x.cuda(), 1, M, K)
        outs = []
        for i in range(depth):
            out = torch.empty(M * N, dtype=torch.bfloat16, device="cuda")
            ttb.check(ttb.cdll.ttb_matmul(cur.data_ptr(), cabi.BFLOAT16, ws_list[i].data_ptr(), cabi.BFLOAT8_B, None, out.data_ptr(),
                                          cabi.BFLOAT16, 1, M, K, N, 0, cabi.MM_DETERMINISTIC | cabi.MM_WORKSPACE_ZEROED | tmem | extra,
                                          ws.data_ptr(), nbytes, None))
            outs.append(out)
            cur = out
        ttb.check(ttb.check_status(None))
        return outs

    plain = chain(0)
    for _ in range(3):
        fast = chain(cabi.MM_WEIGHTS_RESIDENT)
        for a, b in zip(plain, fast):
            assert torch.equal(a, b)
    assert int(ws[:65536].count_nonzero().item()) == 0


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
@pytest.mark.parametrize("M,K,Ns", [(32, 2048, [512, 128, 256]), (64, 1024, [128, 384]), (32, 8192, [1024, 128, 128]), (128, 512, [256, 128]),
                                     (96, 4096, [256, 256, 128, 128])])
def test_several_weights_in_one_launch(ttb, orc, w_dtype, M, K, Ns):
    """ttb_matmul_multi: every output equals the single-weight result (same tolerances against the fp32 reference), with
    per-weight bias, a fused activation, and the scratch left clean for the next launch."""
    import ctypes
    import torch
    x = vectors.randn(41, (M, K), 1.0).bfloat16()
    a = ttb.tilize(x.cuda(), 1, M, K)
    w_devs, w_refs, biases, bias_devs, outs = [], [], [], [], []
    for j, N in enumerate(Ns):
        _, wd, wr = make_case(ttb, orc, 50 + j, M, K, N, w_dtype)
        w_devs.append(wd)
        w_refs.append(wr)
        b = vectors.randn(60 + j, (1, N), 0.5).bfloat16()
        biases.append(b)
        bias_devs.append(ttb.tilize(torch.cat([b, torch.zeros(31, N, dtype=torch.bfloat16)]).cuda(), 1, 32, N) if j != 1 else None)
        outs.append(torch.empty(M * N, dtype=torch.bfloat16, device="cuda"))
    n = len(Ns)
    arr_w = (ctypes.c_void_p * n)(*[t.data_ptr() for t in w_devs])
    arr_b = (ctypes.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in bias_devs])
    arr_o = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
    arr_n = (ctypes.c_int64 * n)(*Ns)
    nbytes = ttb.matmul_multi_workspace_bytes(w_dtype, 1, M, K, n, arr_n)
    ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    for rep in range(2):
        ttb.check(ttb.cdll.ttb_matmul_multi(a.data_ptr(), cabi.BFLOAT16, n, arr_w, w_dtype, arr_b, arr_o, cabi.BFLOAT16, 1, M, K, arr_n,
                                            cabi.ACT_SILU, cabi.MM_WORKSPACE_ZEROED | cabi.MM_WEIGHTS_RESIDENT, ws.data_ptr(), nbytes, None, None, None))
        ttb.check(ttb.check_status(None))
        for j, N in enumerate(Ns):
            y_ref = x.float() @ w_refs[j]
            if j != 1:
                y_ref = y_ref + biases[j].float()
            check(ttb.untilize(outs[j], 1, M, N).reshape(M, N), act_ref(y_ref, cabi.ACT_SILU))
        if nbytes:
            assert int(ws[: min(nbytes, 65536 + (16 << 20))].count_nonzero().item()) == 0


def test_multi_arguments_are_validated(ttb):
    import ctypes
    import torch
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    ns = (ctypes.c_int64 * 2)(128, 96)
    rc = ttb.cdll.ttb_matmul_multi(buf.data_ptr(), cabi.BFLOAT16, 2, ptrs, cabi.BFLOAT8_B, None, ptrs, cabi.BFLOAT16, 1, 288, 64, ns, 0, 0,   # 288 rows: not a decode shape
                                   buf.data_ptr(), 1 << 20, None, None, None)
    assert rc == -3
    rc = ttb.cdll.ttb_matmul_multi(buf.data_ptr(), cabi.BFLOAT16, 5, ptrs, cabi.BFLOAT8_B, None, ptrs, cabi.BFLOAT16, 1, 32, 64, ns, 0, 0,
                                   buf.data_ptr(), 1 << 20, None, None, None)
    assert rc == -1 and b"count" in ttb.cdll.ttb_last_error()
    torch.cuda.synchronize()
    assert int(buf.count_nonzero().item()) == 0


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
@pytest.mark.parametrize("M,K,N", [(32, 512, 256), (32, 4096, 1024), (96, 1024, 384), (32, 4096, 14336), (32, 256, 18944)])
def test_gated_pair_in_one_launch(ttb, orc, w_dtype, M, K, N):
    """MM_GATED: out = silu(a w0 + b0) * (a w1): the gate multiply of the gated MLP formed inside the launch, with and
    without K split over blocks, against fp32 torch on the oracle-unpacked weights; the scratch is clean afterwards and a
    second launch gives the same bytes under a fixed reduction order."""
    import ctypes
    import torch
    x = vectors.randn(71, (M, K), 1.0).bfloat16()
    a = ttb.tilize(x.cuda(), 1, M, K)
    if K * N > 8 << 20:
        (w0, r0), (w1, r1) = (make_big_case(ttb, orc, 72 + j, K, N, w_dtype) for j in range(2))
    else:
        (_, w0, r0), (_, w1, r1) = (make_case(ttb, orc, 72 + j, M, K, N, w_dtype, w_std=0.05) for j in range(2))
    bias = vectors.randn(75, (1, N), 0.5).bfloat16()
    b0 = ttb.tilize(torch.cat([bias, torch.zeros(31, N, dtype=torch.bfloat16)]).cuda(), 1, 32, N)
    out = torch.empty(M * N, dtype=torch.bfloat16, device="cuda")
    arr_w = (ctypes.c_void_p * 2)(w0.data_ptr(), w1.data_ptr())
    arr_b = (ctypes.c_void_p * 2)(b0.data_ptr(), None)
    arr_o = (ctypes.c_void_p * 2)(out.data_ptr(), None)
    arr_n = (ctypes.c_int64 * 2)(N, N)
    nbytes = ttb.matmul_gated_workspace_bytes(w_dtype, 1, M, K, N)
    assert nbytes > 0
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    results = []
    for rep in range(2):
        out.zero_()
        ttb.check(ttb.cdll.ttb_matmul_multi(a.data_ptr(), cabi.BFLOAT16, 2, arr_w, w_dtype, arr_b, arr_o, cabi.BFLOAT16, 1, M, K, arr_n,
                                            cabi.ACT_SILU, cabi.MM_GATED | cabi.MM_WORKSPACE_ZEROED | cabi.MM_DETERMINISTIC, ws.data_ptr(), nbytes,
                                            None, None, None))
        ttb.check(ttb.check_status(None))
        results.append(out.clone())
        assert int(ws[: 65536 + (16 << 20)].count_nonzero().item()) == 0
    assert torch.equal(results[0], results[1])
    xf = x.float().cuda()
    ref = torch.nn.functional.silu(xf @ r0.cuda() + bias.float().cuda()) * (xf @ r1.cuda())
    check(ttb.untilize(results[0], 1, M, N).reshape(M, N), ref)
    # refused where it cannot run: three weights, unequal shapes
    arr_n2 = (ctypes.c_int64 * 2)(N, 128)
    rc = ttb.cdll.ttb_matmul_multi(a.data_ptr(), cabi.BFLOAT16, 2, arr_w, w_dtype, None, arr_o, cabi.BFLOAT16, 1, M, K, arr_n2,
                                   cabi.ACT_SILU, cabi.MM_GATED | cabi.MM_WORKSPACE_ZEROED, ws.data_ptr(), nbytes, None, None, None)
    assert rc == -1


def _plan(ttb, w_dtype, M, K, N, flags=0):
    import ctypes
    out = (ctypes.c_int64 * 5)()
    assert ttb.cdll.ttb_matmul_plan(w_dtype, 1, M, K, N, flags, out, 5) == 0
    return list(out)


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
@pytest.mark.parametrize("M,K,N", [
    (32, 4544, 4672),      # Falcon-7B fused QKV: the last column tile holds 64 columns
    (32, 4544, 4544),      # Falcon-7B dense / selfout
    (32, 18176, 4544),     # Falcon-7B 4h_to_h
    (96, 512, 160),        # 32 columns in the last tile, three tile rows
    (32, 256, 96),         # a single, partial column tile
    (64, 4544, 4672),      # row counts divisible by 64 fall back to one tile row per block
    (256, 512, 160),
])
def test_last_column_tile_of_fewer_than_128_columns(ttb, orc, w_dtype, M, K, N):
    """N a multiple of 32 but not of 128 stays on the tensor-core decode kernel (one launch, decode kind): the missing packed
    tiles of the last column tile read as zeros, no column beyond N is stored - the bytes after the output stay untouched."""
    import torch
    assert _plan(ttb, w_dtype, M, K, N)[:3] == [1, M, 0]
    if K * N > 8 << 20:
        w_dev, w_ref = make_big_case(ttb, orc, 11, K, N, w_dtype, slice_cols=N)
        x = vectors.randn(12, (M, K), 1.0).bfloat16()
    else:
        x, w_dev, w_ref = make_case(ttb, orc, 11, M, K, N, w_dtype)
    a = ttb.tilize(x.cuda(), 1, M, K)
    bias = vectors.randn(13, (1, N), 0.5).bfloat16()
    b_dev = ttb.tilize(torch.cat([bias, torch.zeros(31, N, dtype=torch.bfloat16)]).cuda(), 1, 32, N)
    guard = 4096
    for flags in (0, cabi.MM_OUT_ROW_MAJOR):
        out = torch.full((M * N + guard,), 7.0, dtype=torch.bfloat16, device="cuda")
        nbytes = ttb.matmul_workspace_bytes(w_dtype, 1, M, K, N, flags)
        ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device="cuda")
        ttb.check(ttb.cdll.ttb_matmul(a.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), w_dtype, b_dev.data_ptr(), out.data_ptr(), cabi.BFLOAT16, 1, M, K, N,
                                      cabi.ACT_GELU, flags | cabi.MM_WORKSPACE_ZEROED, ws.data_ptr(), nbytes, None))
        ttb.check(ttb.check_status(None))
        assert bool((out[M * N:] == 7.0).all())
        y = out[: M * N] if flags else ttb.untilize(out[: M * N].clone(), 1, M, N)
        check(y.reshape(M, N), act_ref(x.float().cuda() @ w_ref.cuda() + bias.float().cuda(), cabi.ACT_GELU))
        if nbytes:
            assert int(ws[:65536].count_nonzero().item()) == 0


@pytest.mark.parametrize("M,kinds", [(288, [(256, 0), (32, 0)]), (352, [(256, 0), (96, 0)]), (480, [(256, 0), (224, 0)]),
                                     (544, [(512, 1), (32, 0)]), (736, [(640, 1), (96, 0)])])
def test_row_counts_between_the_kernels_run_as_two_ranges(ttb, orc, M, kinds):
    """Row counts no single tensor-core kernel takes (288-480; above 512 and not a multiple of 128) are served by two launches
    over consecutive row ranges - none of them by the CUDA-core kernel - and match the fp32 reference."""
    import torch
    K, N, w_dtype = 1024, 512, cabi.BFLOAT8_B
    plan = _plan(ttb, w_dtype, M, K, N)
    assert plan[0] == 2 and [(plan[1], plan[2]), (plan[3], plan[4])] == kinds
    assert _plan(ttb, w_dtype, M, K, N, cabi.MM_FORCE_GENERIC)[0] == 0
    x, w_dev, w_ref = make_case(ttb, orc, 21, M, K, N, w_dtype)
    for flags in (0, cabi.MM_A_ROW_MAJOR | cabi.MM_OUT_ROW_MAJOR):
        a = x.cuda().reshape(-1) if flags else ttb.tilize(x.cuda(), 1, M, K)
        y = ttb.matmul(a, w_dev, w_dtype, 1, M, K, N, act=cabi.ACT_RELU, flags=flags, out_fp32=True)
        y = y if flags else ttb.untilize(y, 1, M, N)
        check(y.reshape(M, N), torch.relu(x.float().cuda() @ w_ref.cuda()))


@pytest.mark.parametrize("M,K,N,launches", [(512, 512, 416, 2), (1056, 1024, 4672, 5)])
def test_large_row_counts_with_a_partial_column_tile_run_as_decode_ranges(ttb, orc, M, K, N, launches):
    """What the prefill kernel does not take (N not a multiple of 128) runs as decode launches over ranges of 256 rows - not on
    the CUDA-core kernel - with tiled and with row-major operands, and no byte behind the output is touched."""
    import ctypes
    import torch
    w_dtype = cabi.BFLOAT8_B
    out = (ctypes.c_int64 * 33)()
    assert ttb.cdll.ttb_matmul_plan(w_dtype, 1, M, K, N, 0, out, 33) == 0
    assert out[0] == launches and sum(list(out)[1::2]) == M and not any(list(out)[2::2])
    x, w_dev, w_ref = make_case(ttb, orc, 23, M, K, N, w_dtype)
    ref = torch.relu(x.float().cuda() @ w_ref.cuda())
    for flags in (0, cabi.MM_A_ROW_MAJOR | cabi.MM_OUT_ROW_MAJOR):
        a = x.cuda().reshape(-1) if flags else ttb.tilize(x.cuda(), 1, M, K)
        buf = torch.full((M * N + 4096,), 7.0, dtype=torch.bfloat16, device="cuda")
        nbytes = ttb.matmul_workspace_bytes(w_dtype, 1, M, K, N, flags)
        ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device="cuda")
        ttb.check(ttb.cdll.ttb_matmul(a.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), w_dtype, None, buf.data_ptr(), cabi.BFLOAT16, 1, M, K, N,
                                      cabi.ACT_RELU, flags | cabi.MM_WORKSPACE_ZEROED, ws.data_ptr(), nbytes, None))
        ttb.check(ttb.check_status(None))
        assert bool((buf[M * N:] == 7.0).all())
        y = buf[: M * N] if flags else ttb.untilize(buf[: M * N].clone(), 1, M, N)
        check(y.reshape(M, N), ref)


@pytest.mark.parametrize("M,K,N", [(64, 1024, 37888), (128, 2048, 18944), (256, 1024, 9472)])
def test_many_overlapped_launches_with_two_tile_rows_per_block(ttb, orc, M, K, N):
    """Row counts divisible by 64 run with two tile rows per block; here with several whole-tile rounds per block and dozens of
    launches back to back, each allowed to start while its predecessor drains (the arrangement in which a ring whose
    length was not a multiple of the number of expand teams once lost a barrier phase): no wait runs out, every launch
    gives the first one's bytes, and the result matches the reference."""
    import torch
    assert _plan(ttb, cabi.BFLOAT8_B, M, K, N)[:3] == [1, M, 0]
    w_dev, w_ref = make_big_case(ttb, orc, 31, K, N, cabi.BFLOAT8_B)
    x = vectors.randn(32, (M, K), 1.0).bfloat16()
    a = ttb.tilize(x.cuda(), 1, M, K)
    nbytes = ttb.matmul_workspace_bytes(cabi.BFLOAT8_B, 1, M, K, N, 0)
    ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    outs = [torch.empty(M * N, dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    flags = cabi.MM_WORKSPACE_ZEROED | cabi.MM_WEIGHTS_RESIDENT | cabi.MM_DETERMINISTIC
    for rep in range(3):
        for i in range(16):
            ttb.check(ttb.cdll.ttb_matmul(a.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), cabi.BFLOAT8_B, None, outs[i % 4].data_ptr(), cabi.BFLOAT16,
                                          1, M, K, N, 0, flags, ws.data_ptr(), nbytes, None))
        ttb.check(ttb.check_status(None))
        for o in outs[1:]:
            assert torch.equal(o, outs[0])
    check(ttb.untilize(outs[0], 1, M, N).reshape(M, N), x.float().cuda() @ w_ref.cuda())

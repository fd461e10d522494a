"""The tensor-core projection alone against a float64 product of the same bf16 operands:
token counts from 1 to several tiles, widths that are no multiple of the tile, forced tile
widths, split-K with its in-kernel reduction, and pipelines shorter than the k loop."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run(M, N, K, mode, out_dtype, **force):
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M * 1000003 + N * 1009 + K)
    x = (torch.randn(M, K, device=DEV, generator=g)).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    ref = (x.double() @ w.double().t())
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    if mode == B.GEMM_ADD_RESIDUAL:
        out = torch.randn(M, N, device=DEV, generator=g)
        ref = ref + out.double()
    else:
        out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    ok = B.gemm_tc(x, w, out, M, mode, err, B.stream_ptr(), **force)
    assert ok, "the kernel refused operands it should take"
    torch.cuda.synchronize()
    assert err.item() == 0, B.describe_error_bits(err.item())
    # fp32 accumulation in another order: absolute error of the order of 1e-6 * |terms| summed;
    # a bf16 result adds one rounding, at most 2^-8 relative to the value itself
    scale = (K ** 0.5) * 0.5
    bound = 2e-3 * scale + (2.0 ** -8) * ref.abs() * (out.dtype == torch.bfloat16)
    diff = (out.double() - ref).abs()
    assert torch.isfinite(out).all() and bool((diff <= bound).all()), \
        f"M={M} N={N} K={K} {force}: max diff {diff.max().item():.4g}"
    return out


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 256, 512), (16, 384, 4096), (37, 331, 88), (64, 1000, 200),
                                   (100, 512, 1024), (200, 130, 72), (300, 640, 520), (700, 256, 256)])
def test_shapes(M, N, K):
    from inference_engine_rust_b200.csrc import bindings as B
    run(M, N, K, B.GEMM_STORE, torch.bfloat16)
    run(M, N, K, B.GEMM_STORE, torch.float32)
    run(M, N, K, B.GEMM_ADD_RESIDUAL, torch.float32)


@pytest.mark.parametrize("bt", [16, 32, 64, 128, 256])
def test_every_tile_width(bt):
    from inference_engine_rust_b200.csrc import bindings as B
    run(bt + 3, 300, 392, B.GEMM_STORE, torch.float32, force_bt=bt)
    run(5, 200, 136, B.GEMM_STORE, torch.bfloat16, force_bt=bt)


@pytest.mark.parametrize("splits", [2, 3, 7, 16])
def test_split_k_is_exact_and_repeatable(splits):
    from inference_engine_rust_b200.csrc import bindings as B
    a = run(9, 520, 2048, B.GEMM_STORE, torch.float32, force_splits=splits)
    b = run(9, 520, 2048, B.GEMM_STORE, torch.float32, force_splits=splits)
    assert torch.equal(a, b), "split-K must add its partials in a fixed order"
    run(40, 200, 1096, B.GEMM_ADD_RESIDUAL, torch.float32, force_splits=splits)
    run(3, 4096, 1024, B.GEMM_STORE, torch.bfloat16, force_splits=splits)      # more work items than CTAs


@pytest.mark.parametrize("bt", [64, 128, 256])
@pytest.mark.parametrize("splits", [2, 4, 7])
def test_split_k_with_wide_token_tiles(bt, splits):
    """Many tokens per tile and k in parts: every split adds its share of the tile's rows (four
    rows and four splits per pass), the residual is read with the partials; a ragged last tile,
    a width that is no multiple of 128, a K that is no multiple of 64, and a grid with more work
    items than resident CTAs, where the last split to finish adds the whole tile."""
    from inference_engine_rust_b200.csrc import bindings as B
    a = run(bt + 3, 1000, 1096, B.GEMM_ADD_RESIDUAL, torch.float32, force_bt=bt, force_splits=splits)
    b = run(bt + 3, 1000, 1096, B.GEMM_ADD_RESIDUAL, torch.float32, force_bt=bt, force_splits=splits)
    assert torch.equal(a, b), "the partials must be added in a fixed order"
    run(2 * bt, 392, 1024, B.GEMM_STORE, torch.bfloat16, force_bt=bt, force_splits=splits)
    run(bt - 5, 392, 520, B.GEMM_STORE, torch.float32, force_bt=bt, force_splits=splits)
    run(bt, 128 * 50, 512, B.GEMM_ADD_RESIDUAL, torch.float32, force_bt=bt, force_splits=splits)


def test_short_pipelines_wrap():
    from inference_engine_rust_b200.csrc import bindings as B
    run(24, 300, 4096, B.GEMM_STORE, torch.float32, force_stages=2)
    run(130, 1100, 2048, B.GEMM_STORE, torch.float32, force_stages=3)          # several tiles per CTA


@pytest.mark.parametrize("M,N,K", [(2048, 4096, 192), (2000, 4096, 1024), (1500, 5120, 520), (4096, 4096, 64),
                                   (700, 9000, 136), (2048, 4096, 2560), (1100, 4224, 5128), (300, 20000, 2568),
                                   (2048, 4096, 14336)])
def test_residual_add_over_many_tokens(M, N, K):
    """Residual adds over many tokens: the epilogue hands its tile to TMA, which adds it into the
    residual; with a long k the tiles of the last, partly empty wave are cut into parts of k whose
    products are added in a fixed order (here K = 2,560 and more).  Repeatable to the bit."""
    from inference_engine_rust_b200.csrc import bindings as B
    a = run(M, N, K, B.GEMM_ADD_RESIDUAL, torch.float32)
    b = run(M, N, K, B.GEMM_ADD_RESIDUAL, torch.float32)
    assert torch.equal(a, b), "two identical runs differ"
    sc = B.GemmScratch.get(a.device)
    assert int(sc.counters.abs().sum()) == 0, "a tile's flag was left raised"


def test_token_tiles_walked_in_groups():
    """Activations above 64 MB: the token tiles are walked in groups sized for the L2 (another
    order of the tiles, the same products).  Weight-major with the residual add (k of 14,336, the
    last wave cut into parts), token-major store, and the gated form; repeatable to the bit."""
    from inference_engine_rust_b200.csrc import bindings as B
    a = run(2400, 256, 14336, B.GEMM_ADD_RESIDUAL, torch.float32)
    b = run(2400, 256, 14336, B.GEMM_ADD_RESIDUAL, torch.float32)
    assert torch.equal(a, b)
    a = run(8400, 384, 4096, B.GEMM_STORE, torch.bfloat16)
    b = run(8400, 384, 4096, B.GEMM_STORE, torch.bfloat16)
    assert torch.equal(a, b)
    run(8400, 1280, 4096, B.GEMM_ADD_RESIDUAL, torch.float32)
    run(2400, 4096, 14336, B.GEMM_ADD_RESIDUAL, torch.float32)     # 10 token tiles x 32 row tiles in 3 groups
    # gated: 8,400 tokens x 4,096 is 69 MB of activations
    M, I, K = 8400, 384, 4096
    g = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV, generator=g) * (2.0 / K ** 0.5)).bfloat16()
    act = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert B.gemm_tc_gated(x, w, act, M, err, B.stream_ptr())
    torch.cuda.synchronize()
    assert err.item() == 0
    gate = x.double() @ w[:I].double().t()
    up = x.double() @ w[I:].double().t()
    ref = gate * torch.sigmoid(gate) * up
    bound = 1e-3 + (2.0 ** -8) * ref.abs() + 1e-3 * (gate.abs() + 1) * up.abs()
    assert torch.isfinite(act).all() and bool(((act.double() - ref).abs() <= bound).all())


def test_many_tiles_per_cta():
    from inference_engine_rust_b200.csrc import bindings as B
    run(1500, 4096, 256, B.GEMM_STORE, torch.bfloat16)                         # 32 x 6 tiles on 148 CTAs
    run(33, 40000, 128, B.GEMM_STORE, torch.float32)                           # 313 thin tiles


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 1000, 264), (700, 640, 520), (2048, 384, 128)])
def test_token_major_kernel_in_every_mode(M, N, K):
    """Prompts: 128 tokens on the MMA's M side, 256 weight rows per tile; store (the default for
    many tokens) and, forced, the residual add."""
    from inference_engine_rust_b200.csrc import bindings as B
    run(M, N, K, B.GEMM_STORE, torch.bfloat16)
    run(M, N, K, B.GEMM_STORE, torch.float32)
    run(M, N, K, B.GEMM_ADD_RESIDUAL, torch.float32, force_stages=-1)


@pytest.mark.parametrize("M", [65, 96, 128, 129, 200, 256, 257, 300, 384, 385, 512, 513])
def test_between_decoding_and_prompts_at_layer_sizes(M):
    """65 to 513 tokens at the widths of a 7B layer, with the tile and the splits the kernel
    chooses itself there (64-, 128- and 256-token tiles, split over k while the tiles alone leave
    SMs empty; token-major stores from 257 tokens on)."""
    from inference_engine_rust_b200.csrc import bindings as B
    run(M, 6144, 4096, B.GEMM_STORE, torch.bfloat16)
    run(M, 4096, 4096, B.GEMM_ADD_RESIDUAL, torch.float32)
    run(M, 4096, 14336, B.GEMM_ADD_RESIDUAL, torch.float32)


def test_refuses_what_tma_cannot_load():
    from inference_engine_rust_b200.csrc import bindings as B
    x = torch.randn(4, 100, device=DEV).bfloat16()
    w = torch.randn(64, 100, device=DEV).bfloat16()
    out = torch.empty(4, 64, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert B.gemm_tc(x, w, out, 4, B.GEMM_STORE, err, B.stream_ptr()) is False     # K = 100 is no multiple of 8


def test_row_results_do_not_depend_on_the_batch():
    """A token's projection is the same alone, among 7 others, and in a prompt of hundreds,
    up to the rounding of split-K partial sums."""
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(300, 1024, device=DEV, generator=g).bfloat16()
    w = torch.randn(768, 1024, device=DEV, generator=g).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = []
    for M in (1, 8, 300):
        out = torch.empty(M, 768, device=DEV)
        assert B.gemm_tc(x, w, out, M, B.GEMM_STORE, err, B.stream_ptr())
        outs.append(out[0].clone())
    assert torch.allclose(outs[0], outs[1], atol=1e-3, rtol=1e-4) and torch.allclose(outs[0], outs[2], atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("M,I,K", [(1, 128, 64), (8, 200, 136), (40, 160, 96), (100, 384, 512), (300, 1000, 264),
                                   (64, 14336, 256), (8, 14336, 512), (33, 9600, 128)])
def test_gated_product_is_silu_gate_times_up(M, I, K):
    """The fused feed-forward entry: two accumulators per tile, activation in the epilogue."""
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M + I + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV, generator=g) * (2.0 / K ** 0.5)).bfloat16()
    act = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    forces = [{}, {"force_stages": 2}, {"force_bt": 128}]
    # the decoding form (weight rows on the MMA's M side) at every token tile that holds M
    forces += [{"force_bt": bt} for bt in (16, 32, 64) if M <= bt] + ([{"force_bt": 64, "force_stages": 2}] if M <= 64 else [])
    for force in forces:
        act.fill_(float("nan"))
        assert B.gemm_tc_gated(x, w, act, M, err, B.stream_ptr(), **force)
        torch.cuda.synchronize()
        assert err.item() == 0
        gate = x.double() @ w[:I].double().t()
        up = x.double() @ w[I:].double().t()
        ref = gate * torch.sigmoid(gate) * up
        diff = (act.double() - ref).abs()
        bound = 1e-3 + (2.0 ** -8) * ref.abs() + 1e-3 * (gate.abs() + 1) * up.abs()
        assert torch.isfinite(act).all() and bool((diff <= bound).all()), f"{force}: max diff {diff.max().item():.4g}"


# ---- one-token steps of 17 to 64 tokens: an RMSNorm split around the kernel boundary ---------------


@pytest.mark.parametrize("M,N,K", [(17, 4096, 4096), (32, 4096, 14336), (64, 4096, 4096), (40, 520, 2048)])
@pytest.mark.parametrize("wdt", [torch.bfloat16, torch.float32])
def test_split_k_residual_add_writes_the_next_norms_first_half(M, N, K, wdt):
    """Beside the new residual rows the split-K reduction writes bf16(row x scale vector) and one sum of
    squares per row and tile of 128 columns; repeatable to the bit; refused where nothing is split."""
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    nw = (1.0 + 0.1 * torch.randn(N, device=DEV, generator=g)).to(wdt)
    res0 = torch.randn(M, N, device=DEV, generator=g)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    tiles = -(-N // 128)
    outs = []
    for _ in range(2):
        out = res0.clone()
        scaled = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        sumsq = torch.full((M, tiles), float("nan"), device=DEV)
        ahead = B.norm_ahead(nw, scaled, sumsq)
        assert B.gemm_tc_scaled(x, w, out, M, B.GEMM_ADD_RESIDUAL, err, B.stream_ptr(), ahead=ahead)
        torch.cuda.synchronize()
        assert err.item() == 0 and ahead.parts == tiles
        ref = x.double() @ w.double().t() + res0.double()
        assert bool(((out.double() - ref).abs() <= 2e-3 * (K ** 0.5) * 0.5).all())
        assert torch.equal(scaled, (out * nw.float()).bfloat16())
        pad = torch.zeros(M, tiles * 128, device=DEV, dtype=torch.float64)
        pad[:, :N] = out.double()
        assert torch.allclose(sumsq.double(), (pad.view(M, tiles, 128) ** 2).sum(-1), rtol=1e-5, atol=1e-6)
        outs.append((out, scaled, sumsq))
    assert all(torch.equal(a, b) for a, b in zip(*outs))
    ahead = B.norm_ahead(nw, scaled, sumsq)
    assert not B.gemm_tc_scaled(x, w, res0.clone(), M, B.GEMM_ADD_RESIDUAL, err, B.stream_ptr(), ahead=ahead, force_splits=1)


@pytest.mark.parametrize("M,N,K,parts", [(17, 6144, 4096, 32), (64, 6144, 4096, 32), (33, 520, 2048, 1), (64, 4096, 4096, 7)])
def test_split_k_store_applies_the_norms_second_half(M, N, K, parts):
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M * 3 + N + K + parts)
    rows = torch.randn(M, K, device=DEV, generator=g) * 3.0
    nw = 1.0 + 0.1 * torch.randn(K, device=DEV, generator=g)
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    eps = 1e-5
    scaled = (rows * nw).bfloat16()
    per = -(-K // parts)
    pad = torch.zeros(M, per * parts, device=DEV, dtype=torch.float64)
    pad[:, :K] = rows.double()
    sumsq = (pad.view(M, parts, per) ** 2).sum(-1).float().contiguous()
    rstd = 1.0 / torch.sqrt((rows.double() ** 2).mean(-1, keepdim=True) + eps)
    ref = (scaled.double() * rstd) @ w.double().t()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = B.RowScale(sumsq=sumsq.data_ptr(), parts=parts, hidden=K, eps=eps)
    for odt in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=odt)
        assert B.gemm_tc_scaled(scaled, w, out, M, B.GEMM_STORE, err, B.stream_ptr(), scale=scale)
        torch.cuda.synchronize()
        assert err.item() == 0
        bound = 2e-3 * (K ** 0.5) * 0.5 + 1e-5 * ref.abs() + (2.0 ** -8) * ref.abs() * (odt == torch.bfloat16)
        diff = (out.double() - ref).abs()
        assert torch.isfinite(out).all() and bool((diff <= bound).all()), f"{odt}: max diff {diff.max().item():.4g}"


def test_a_wait_between_ctas_that_runs_out_is_reported_and_harmless():
    """The splits of a tile wait for one another on the tile's counter, with a limit.  Here the counter of
    one tile is set so that its splits can never all be counted in (and the limit is shortened, so that the
    test takes milliseconds): the kernel ends by itself, the device error word says that a wait expired, the
    other tile's result is right, and after the counter is put back the next launch is right everywhere."""
    from inference_engine_rust_b200.csrc import bindings as B
    M, N, K, splits = 8, 256, 2048, 4                      # two tiles of 128 rows, four splits each: 8 CTAs
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    ref = x.double() @ w.double().t()
    bound = 2e-3 * (K ** 0.5) * 0.5
    sc = B.GemmScratch.get(torch.device(DEV))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    assert int(sc.counters[:2].abs().sum()) == 0, "counters are zero between launches"
    B.gemm_tc_set_poll_limit(1 << 12)
    try:
        sc.counters[0] = -1000                             # tile 0: never reaches 4
        out = torch.full((M, N), float("nan"), device=DEV)
        assert B.gemm_tc(x, w, out, M, B.GEMM_STORE, err, B.stream_ptr(), force_splits=splits)
        torch.cuda.synchronize()
        assert err.item() & B.ERR_WAIT_EXPIRED, "the expired wait was not reported"
        assert torch.isnan(out[:, :128]).all(), "tile 0 must not have been written from partial sums"
        assert bool(((out[:, 128:].double() - ref[:, 128:]).abs() <= bound).all()), "tile 1 is independent of tile 0"
    finally:
        B.gemm_tc_set_poll_limit(0)
        sc.counters.zero_()
        err.zero_()
    out = torch.full((M, N), float("nan"), device=DEV)
    assert B.gemm_tc(x, w, out, M, B.GEMM_STORE, err, B.stream_ptr(), force_splits=splits)
    torch.cuda.synchronize()
    assert err.item() == 0
    assert bool(((out.double() - ref).abs() <= bound).all())
    assert int(sc.counters[:2].abs().sum()) == 0

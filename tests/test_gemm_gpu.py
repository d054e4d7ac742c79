"""GPU parity of the tcgen05 GEMM with the oracle, called through the C ABI (pg_hgemm_ex).

Every case (tests/helpers.py:check_gemm): the acceptance bound max|C - C_ref| <= (2e-2 * sqrt(k/4096) + eps_out) *
max|C_ref| (C_ref = fp32-accumulated product of the same 16-bit inputs; eps_out = one rounding step of the output
type); per element, C must be the correctly rounded value of a number within the fp32 accumulation slack of the oracle's
sum; and, where the exact k-ordered oracle is affordable, the reference test's own bound 0.5*k/4096.  Inputs are generated on the CPU from fixed seeds, C is
pre-filled with garbage (the reference's tests do the same: test/test_gemm.py:32-34).
"""
import pytest
import torch

import oracle
from tests import helpers

pytestmark = pytest.mark.gpu

BF16, F16 = torch.bfloat16, torch.float16


def run_case(m, n, k, dtype, variant, block_n, seed=0, gen=oracle.gemm_inputs_uniform, exact=None):
    from peakgemm_b200 import capi

    a, b = gen(m, n, k, dtype, seed)
    c = helpers.garbage_like((m, n), dtype, "cuda")
    capi.hgemm(c, a.cuda(), b.cuda(), variant=variant, block_n=block_n)
    torch.cuda.synchronize()
    assert capi.device_status() == 0, "a kernel abandoned a bounded wait"
    return helpers.check_gemm(c, a, b, exact_rows=exact)


# ---- the smallest end-to-end case first: if this fails nothing else is worth running
def test_single_tile_one_cta(cuda):
    run_case(128, 256, 64, BF16, 1, 256)


def test_single_tile_multi_kblock(cuda):
    run_case(128, 256, 512, BF16, 1, 256)


@pytest.mark.parametrize("block_n", [64, 128, 256])
@pytest.mark.parametrize("dtype", [BF16, F16])
def test_one_cta_variants(cuda, block_n, dtype):
    run_case(512, 768, 1024, dtype, 1, block_n, seed=1)


def test_pair_single_tile(cuda):
    run_case(256, 256, 64, BF16, 2, 256)


def test_pair_multi_kblock(cuda):
    run_case(256, 256, 1024, BF16, 2, 256)


@pytest.mark.parametrize("block_n", [64, 128, 256])
@pytest.mark.parametrize("dtype", [BF16, F16])
def test_pair_variants(cuda, block_n, dtype):
    run_case(512, 768, 1024, dtype, 2, block_n, seed=1)


# ---- CTA pair with two row blocks per CTA (variant 5): 512 x 256 tiles, both accumulators belong to one tile
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("m,n,k", [
    (512, 256, 64),        # one tile, one k-block
    (512, 256, 1024),      # one tile, the ring wraps four times
    (1024, 768, 512),      # 2 x 3 tiles
    (4096, 8192, 256),     # 256 tiles on 74 pairs: several tiles per pair, both accumulators drained and refilled
    (300, 264, 136),       # tails in m (the second row block is partly empty), n and k
    (260, 520, 72),        # the second row block holds 4 rows
    (128, 256, 128),       # fewer rows than one row block of the peer CTA
    (1000, 1000, 1000),
])
def test_pair_two_row_blocks(cuda, m, n, k, dtype):
    run_case(m, n, k, dtype, 5, 0, seed=21, exact=True)


def test_pair_two_row_blocks_matches_pair_kernel_bitwise(cuda):
    """The same k-ordered accumulation per element as the 256 x 256 CTA-pair kernel: identical bits."""
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_uniform(2048, 2304, 4096, BF16, 22)
    ad, bd = a.cuda(), b.cuda()
    c2 = helpers.garbage_like((2048, 2304), BF16, "cuda")
    c5 = helpers.garbage_like((2048, 2304), BF16, "cuda")
    capi.hgemm(c2, ad, bd, variant=2, block_n=256)
    capi.hgemm(c5, ad, bd, variant=5)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.equal(c2.view(torch.int16), c5.view(torch.int16))
    assert capi.lib().pg_hgemm_ex(ad.data_ptr(), ad.data_ptr(), ad.data_ptr(), 512, 256, 64, 64, 64, 256, 1, 5, 128,
                                  0, None) == 1      # variant 5 exists at block_n 256 only


# ---- pair split-K (variant 6, 64 < m <= 128): a CTA pair per 128 x 256 or 128 x 128 tile (2-CTA MMA at M = 128, 64 rows
# of A per CTA), 1 or 2 pairs over k per cluster, partial sums through distributed shared memory
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("m,n,k,block_n", [
    (128, 256, 64, 256),      # one tile, one k-block: one pair
    (128, 256, 4096, 256),    # one tile, 2 pairs over k
    (128, 256, 4096, 128),    # two 128-wide tiles, 2 pairs each
    (128, 4096, 4096, 0),     # benchmark config 3 shape: automatic width and pairs
    (128, 8192, 2048, 0),
    (128, 14336, 1024, 0),    # 56 tiles of 256, one pair each
    (100, 520, 1000, 256),    # tails in m, n and k; the last k-block ragged
    (100, 520, 1000, 128),
    (65, 264, 448, 0),        # 7 k-blocks: too few for 2 pairs; one row in the second CTA
    (96, 2048, 1152, 256),    # 18 k-blocks over 2 pairs
    (128, 512, 832, 128),     # 13 k-blocks over 2 pairs: uneven slices
    # 256-row tiles (128 rows of A per CTA, the ordinary M = 256 pair MMA) for m > 128
    (256, 256, 4096, 256),    # one tile, 2 pairs over k
    (512, 4096, 4096, 0),     # 32 tiles x 2 pairs
    (384, 4096, 2048, 0),     # the second tile row half empty
    (300, 520, 1000, 128),    # tails in m, n and k
    (512, 2048, 832, 256),    # 13 k-blocks over 2 pairs
    (129, 264, 64, 0),        # one k-block: one pair; a single row in the second CTA
])
def test_pair_split_k(cuda, m, n, k, block_n, dtype):
    run_case(m, n, k, dtype, 6, block_n, seed=24, exact=True)


def test_pair_split_k_is_deterministic_and_refuses_other_shapes(cuda):
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_llm(128, 4096, 14336, BF16, 25)
    ad, bd = a.cuda(), b.cuda()
    outs = []
    for _ in range(3):
        c = helpers.garbage_like((128, 4096), BF16, "cuda")
        capi.hgemm(c, ad, bd, variant=6)
        outs.append(c)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    helpers.check_gemm(outs[0], a, b, exact_rows=False)
    p = ad.data_ptr()
    assert capi.lib().pg_hgemm_ex(p, p, p, 128, 128256, 64, 64, 64, 128256, 1, 6, 0, 0, None) == 1  # too many tiles
    assert capi.lib().pg_hgemm_ex(p, p, p, 8192, 8192, 64, 64, 64, 8192, 1, 6, 0, 0, None) == 1
    assert capi.lib().pg_hgemm_ex(p, p, p, 128, 256, 64, 64, 64, 256, 1, 6, 64, 0, None) == 1       # block_n


# ---- cluster split-K (variant 3): 2, 4 or 8 CTAs share a tile and combine partial sums through
# distributed shared memory.  The shapes steer the planner to every cluster size and slice width.
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("m,n,k,block_n", [
    (64, 128, 2048, 64),      # 2 tiles  -> S=8, 8 columns per CTA
    (64, 128, 2048, 128),     # 1 tile   -> S=8, 16 columns per CTA
    (128, 1024, 1024, 128),   # 8 tiles  -> S=8
    (16, 4096, 4096, 0),      # benchmark config 3 shape: 32 tiles of 128 -> S=4
    (128, 4096, 1024, 64),    # 64 tiles -> S=2
    (100, 520, 1000, 0),      # tails in m, n and k
    (64, 2048, 576, 128),     # 9 k-blocks over S=4: the last CTA's slice is empty
    (200, 264, 8192, 64),     # two tile rows
])
def test_split_k_cluster(cuda, m, n, k, block_n, dtype):
    run_case(m, n, k, dtype, 3, block_n, seed=6)


def test_split_k_is_deterministic_and_refuses_unsplittable_shapes(cuda):
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_uniform(128, 4096, 14336, BF16, 7)
    ad, bd = a.cuda(), b.cuda()
    outs = []
    for _ in range(3):
        c = torch.empty(128, 4096, dtype=BF16, device="cuda")
        capi.hgemm(c, ad, bd, variant=3)
        outs.append(c)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    helpers.check_gemm(outs[0], a, b, exact_rows=False)
    p = ad.data_ptr()
    # k too short to split, and a shape with more tiles than SMs
    assert capi.lib().pg_hgemm_ex(p, p, p, 128, 64, 64, 64, 64, 64, 1, 3, 0, 0, None) == 1
    assert capi.lib().pg_hgemm_ex(p, p, p, 8192, 8192, 8192, 8192, 8192, 8192, 1, 3, 0, 0, None) == 1


# ---- skinny kernel (variant 4, m <= 64): operands swapped, optional cluster split-K over k.
# n = 128 * tiles steers the cluster size.  Up to 16 tokens (two CTAs per SM, 296 slots): 16 and 32 tiles -> S=8,
# 64 -> 4, 112 -> 2, >= 163 -> 1.  17-64 tokens: 16 tiles -> S=8, 32 -> 4, 64 -> 2, >= 128 -> 1 with one CTA per SM and
# the deep pipeline; 17-32 tokens and more than 148 tiles: two CTAs per SM, short pipeline, no receive buffer; 17-32
# tokens and 82-162 tiles: two CTAs per SM with S=2.
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("m,n,k", [
    (16, 2048, 2048),      # S=8, 16 rows per CTA
    (1, 2048, 4096),       # a single token
    (16, 4096, 4096),      # S=8 (benchmark config 3)
    (17, 4096, 1024),      # 32-token tile, S=4
    (33, 8192, 512),       # 64-token tile, S=2
    (64, 8192, 4096),      # full 64-token tile
    (16, 14336, 4096),     # S=2, 224 CTAs on 148 SMs
    (7, 1000, 264),        # tails in n and k, too few k-blocks to split
    (16, 128, 64),         # one CTA, one k-block
    (48, 16384 + 8, 192),  # 129 CTAs of the deep 64-token pipeline, ragged last tile
    (12, 21000, 1024),     # 16-token tile, S=1, no receive buffer: 165 CTAs, two per SM, the ring wraps twice
    (24, 19208, 448),      # 32-token tile, two CTAs per SM (151 tiles), ragged last tile, ring wraps
    (48, 20000, 704),      # 64-token tile, 157 CTAs on 148 SMs
    (24, 14336, 1024),     # 32-token tile, one wave of 112 tiles: two CTAs per SM, k split in two, ring of 4 wraps
])
def test_skinny_kernel(cuda, m, n, k, dtype):
    run_case(m, n, k, dtype, 4, 0, seed=8, gen=oracle.gemm_inputs_llm)


def test_skinny_refuses_large_m_and_is_deterministic(cuda):
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_llm(16, 4096, 14336, BF16, 9)
    ad, bd = a.cuda(), b.cuda()
    outs = []
    for _ in range(3):
        c = helpers.garbage_like((16, 4096), BF16, "cuda")
        capi.hgemm(c, ad, bd)                 # automatic choice for m <= 64
        outs.append(c)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    helpers.check_gemm(outs[0], a, b, exact_rows=False)
    p = ad.data_ptr()
    assert capi.lib().pg_hgemm_ex(p, p, p, 65, 64, 64, 64, 64, 64, 1, 4, 0, 0, None) == 1


# ---- persistence: more tiles than CTAs, several tiles per CTA, both accumulators reused
@pytest.mark.parametrize("variant,block_n", [(1, 64), (1, 256), (2, 64), (2, 256)])
def test_many_tiles_per_cta(cuda, variant, block_n):
    run_case(2048, 4096, 256, BF16, variant, block_n, seed=2, exact=True)


# ---- tails the reference never validates (it reads out of bounds there): TMA zero-fill / clipping
@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("m,n,k", [
    (16, 64, 64), (1, 8, 8), (130, 72, 40), (127, 248, 1000), (257, 264, 72), (300, 520, 136),
    (128, 256, 8), (384, 8, 4096),
])
def test_tails(cuda, variant, m, n, k):
    run_case(m, n, k, BF16, variant, 0 if variant == 1 else 128, seed=3)


def test_empty_and_k0(cuda):
    from peakgemm_b200 import capi

    a = torch.zeros(0, 64, dtype=BF16, device="cuda")
    b = torch.zeros(64, 64, dtype=BF16, device="cuda")
    c = torch.zeros(0, 64, dtype=BF16, device="cuda")
    capi.hgemm(c, a, b)                       # m == 0: no-op
    a = torch.zeros(32, 0, dtype=BF16, device="cuda")
    b = torch.zeros(64, 0, dtype=BF16, device="cuda")
    c = helpers.garbage_like((32, 64), BF16, "cuda")
    st = capi.lib().pg_hgemm(c.data_ptr(), 0, 0, 32, 64, 0, 0, 0, 64, capi.PG_BF16, None)
    assert st == 0
    torch.cuda.synchronize()
    assert (c == 0).all()                     # k == 0: an empty sum


def test_ldc_column_block(cuda):
    """ldc > n: a column block written in place into a wider C (what the column-sharded caller does)."""
    from peakgemm_b200 import capi

    m, n, k, n_full = 384, 256, 512, 1024
    a, b = oracle.gemm_inputs_uniform(m, n, k, BF16, 5)
    full = helpers.garbage_like((m, n_full), BF16, "cuda")
    before = full.clone()
    block = full[:, 512:512 + n]
    capi.hgemm(block, a.cuda(), b.cuda(), ldc=n_full)
    torch.cuda.synchronize()
    helpers.check_gemm(block, a, b)
    assert torch.equal(full[:, :512], before[:, :512]) and torch.equal(full[:, 768:], before[:, 768:])


def test_multi_destination_epilogue(cuda):
    """pg_hgemm_multi on one GPU: three local buffers stand in for the peers' C; each must receive the block."""
    from peakgemm_b200 import capi

    m, n, k, n_full = 600, 512, 1024, 1536
    a, b = oracle.gemm_inputs_uniform(m, n, k, BF16, 12)
    fulls = [helpers.garbage_like((m, n_full), BF16, "cuda") for _ in range(3)]
    before = fulls[1].clone()
    ptrs = [f[:, 512:512 + n].data_ptr() for f in fulls]
    capi.hgemm_multi(ptrs, a.cuda(), b.cuda(), ldc=n_full)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    helpers.check_gemm(fulls[0][:, 512:512 + n], a, b)
    for f in fulls[1:]:
        assert torch.equal(f[:, 512:512 + n], fulls[0][:, 512:512 + n])
    assert torch.equal(fulls[1][:, :512], before[:, :512]) and torch.equal(fulls[1][:, 1024:], before[:, 1024:])
    # enough tiles for the 256-wide CTA-pair kernel, several tiles per CTA pair (the staging boxes are reused
    # across tiles while stores to three destinations are in flight), tails in m and n
    m3, n3, k3 = 4000, 4104, 320
    a3, b3 = oracle.gemm_inputs_uniform(m3, n3, k3, BF16, 14)
    outs3 = [helpers.garbage_like((m3, n3), BF16, "cuda") for _ in range(3)]
    capi.hgemm_multi([o.data_ptr() for o in outs3], a3.cuda(), b3.cuda(), ldc=n3)
    single = helpers.garbage_like((m3, n3), BF16, "cuda")
    capi.hgemm(single, a3.cuda(), b3.cuda())
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    helpers.check_gemm(outs3[0], a3, b3, exact_rows=False)
    for o in outs3:
        assert torch.equal(o, single)
    # a shape of the 512 x 256 kernel (208 large tiles, three waves), tails in m and n
    m5, n5, k5 = 8000, 3304, 136
    assert capi.hgemm_config(m5, n5, k5) == (5, 256)
    a5, b5 = oracle.gemm_inputs_uniform(m5, n5, k5, BF16, 15)
    outs5 = [helpers.garbage_like((m5, n5), BF16, "cuda") for _ in range(3)]
    capi.hgemm_multi([o.data_ptr() for o in outs5], a5.cuda(), b5.cuda(), ldc=n5)
    single5 = helpers.garbage_like((m5, n5), BF16, "cuda")
    capi.hgemm(single5, a5.cuda(), b5.cuda())
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    rows5 = torch.arange(64) * 125
    helpers.check_gemm(outs5[0][rows5.cuda()], a5[rows5], b5, exact_rows=False)
    for o in outs5:
        assert torch.equal(o, single5)
    # a small-m case takes the one-CTA kernel
    a2, b2 = oracle.gemm_inputs_uniform(48, 256, 512, F16, 13)
    outs = [helpers.garbage_like((48, 256), F16, "cuda") for _ in range(2)]
    capi.hgemm_multi([o.data_ptr() for o in outs], a2.cuda(), b2.cuda(), ldc=256)
    torch.cuda.synchronize()
    helpers.check_gemm(outs[0], a2, b2)
    assert torch.equal(outs[0], outs[1])
    L = capi.lib()
    assert L.pg_hgemm_multi(None, 1, 0, 0, 8, 8, 8, 8, 8, 8, 1, 0, None) == 1
    import ctypes
    arr = (ctypes.c_void_p * 9)(*[ctypes.c_void_p(outs[0].data_ptr())] * 9)
    assert L.pg_hgemm_multi(arr, 9, outs[0].data_ptr(), outs[0].data_ptr(), 8, 8, 8, 8, 8, 8, 1, 0, None) == 1


def test_argument_errors(cuda):
    from peakgemm_b200 import capi

    L = capi.lib()
    a = torch.zeros(128, 64, dtype=BF16, device="cuda")
    p = a.data_ptr()
    assert L.pg_hgemm(p, p, p, 128, 12, 64, 64, 64, 12, 1, None) == 3      # n % 8
    assert L.pg_hgemm(p, p, p, 128, 64, 12, 12, 12, 64, 1, None) == 3      # k % 8
    assert L.pg_hgemm(p + 2, p, p, 128, 64, 64, 64, 64, 64, 1, None) == 2  # misaligned
    assert L.pg_hgemm(None, p, p, 128, 64, 64, 64, 64, 64, 1, None) == 1   # null
    assert L.pg_hgemm(p, p, p, -1, 64, 64, 64, 64, 64, 1, None) == 1
    assert L.pg_hgemm(p, p, p, 128, 64, 64, 64, 64, 64, 7, None) == 1      # dtype
    assert L.pg_hgemm_ex(p, p, p, 128, 64, 64, 64, 64, 64, 1, 1, 96, 0, None) == 1  # block_n


# ---- the benchmark configurations
def test_config1_bf16_2048(cuda):
    """bf16 m=n=k=2048, U[-1,1], seed 0, automatic configuration, exact oracle too."""
    err, tol = run_case(2048, 2048, 2048, BF16, 0, 0, seed=0, exact=True)
    assert err <= 0.5  # pure bf16 output rounding at |C| <= 128 is <= 0.25


@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("size", [2048, 4096])
def test_config2_square(cuda, size, dtype):
    run_case(size, size, size, dtype, 0, 0, seed=1, exact=(size <= 2048))


@pytest.mark.parametrize("dtype", [BF16, F16])
def test_config2_8192_vs_device_oracle(cuda, dtype):
    """Full size of the headline shape: every element against the device restatement of the
    reference's naive kernel, and 64 sampled rows against the CPU oracle."""
    from peakgemm_b200 import capi

    s = 8192
    a, b = oracle.gemm_inputs_uniform(s, s, s, dtype, 1)
    ad, bd = a.cuda(), b.cuda()
    c = helpers.garbage_like((s, s), dtype, "cuda")
    capi.hgemm(c, ad, bd)
    ref = helpers.gemm_naive_device(ad, bd)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    diff = (c.float() - ref.float()).abs().max().item()
    assert diff <= oracle.reference_abs_tolerance(s), diff
    rows = torch.arange(0, s, s // 64) + 7
    helpers.check_gemm(c[rows], a[rows], b, exact_rows=False)


def full_size_case(m, n, k, dtype, seed, gen, sample_rows=64, exact_rows=4, workspace=True):
    """A full-size benchmark shape the way the operator runs it (automatic configuration, tail-split workspace
    when the shape qualifies): every element against the device restatement of the reference's naive kernel,
    `sample_rows` rows against the CPU oracle (acceptance bound + per-element rounding check) and `exact_rows` of
    them against the exact k-ordered CPU sum."""
    from peakgemm_b200 import capi

    a, b = gen(m, n, k, dtype, seed)
    ad, bd = a.cuda(), b.cuda()
    c = helpers.garbage_like((m, n), dtype, "cuda")
    need = capi.hgemm_workspace_bytes(m, n, k) if workspace else 0
    ws = torch.full((need,), 0xAB, dtype=torch.uint8, device="cuda") if need else None
    capi.hgemm_ws(c, ad, bd, ws)
    torch.cuda.synchronize()
    assert capi.device_status() == 0, "a kernel abandoned a bounded wait"
    helpers.check_gemm_device(c, ad, bd)
    rows = (torch.arange(sample_rows) * (m // sample_rows) + 7 * (m > 7 * sample_rows)) % m if m > sample_rows \
        else torch.arange(m)
    helpers.check_gemm(c[rows.cuda()], a[rows], b, exact_rows=False)
    ex = rows[:exact_rows]
    helpers.check_gemm(c[ex.cuda()], a[ex], b, exact_rows=True)
    return need


@pytest.mark.parametrize("dtype", [BF16, F16])
def test_config2_16384(cuda, dtype):
    """benchmark config 2 at its largest size (the reference validates it too: test/cpp/test_gemm_half.cpp:174-192).
    The automatic choice is the CTA-pair kernel with 512 x 256 tiles: 2048 tiles, 27.7 waves on 74 SM pairs."""
    full_size_case(16384, 16384, 16384, dtype, 1, oracle.gemm_inputs_uniform)


@pytest.mark.parametrize("m", [16, 128, 1024])
@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336)])
def test_config3_skinny(cuda, m, n, k):
    run_case(m, n, k, BF16, 0, 0, seed=2, gen=oracle.gemm_inputs_llm, exact=False)


@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)])
def test_config3_m4096(cuda, n, k):
    """benchmark config 3 at m = 4096, all four (n, k)."""
    full_size_case(4096, n, k, BF16, 2, oracle.gemm_inputs_llm, sample_rows=32)


@pytest.mark.parametrize("m", [16, 128, 1024])
def test_config3_vocab_projection(cuda, m):
    """benchmark config 3 at (n, k) = (128256, 4096) for the remaining m (m = 4096: test_config3_m4096)."""
    full_size_case(m, 128256, 4096, BF16, 2, oracle.gemm_inputs_llm, sample_rows=16)


def test_config5_per_rank_block(cuda):
    """benchmark config 5 as one of 8 ranks sees it: m = 32768, k = 16384, its 4096 columns of B (seed 4), written
    as a column block into a wider C (ldc > n) the way the column-sharded caller does."""
    from peakgemm_b200 import capi

    m, n_local, k, ldc = 32768, 4096, 16384, 8192
    g = torch.Generator().manual_seed(4)
    a = (torch.rand(m, k, generator=g) * 2 - 1).to(BF16)
    b = (torch.rand(n_local, k, generator=g) * 2 - 1).to(BF16)       # the first rank's rows of B
    ad, bd = a.cuda(), b.cuda()
    wide = helpers.garbage_like((m, ldc), BF16, "cuda")
    before = wide[:, :n_local].clone()
    block = wide[:, n_local:]
    capi.hgemm(block, ad, bd, ldc=ldc)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.equal(wide[:, :n_local], before), "columns outside the block were written"
    helpers.check_gemm_device(block, ad, bd)
    rows = torch.arange(32) * 1024 + 11
    helpers.check_gemm(block[rows.cuda()], a[rows], b, exact_rows=False)
    helpers.check_gemm(block[rows[:4].cuda()], a[rows[:4]], b, exact_rows=True)


# ---- size-independent properties at full size
def test_linearity_in_a(cuda):
    """(2A) B^T == 2 (A B^T) exactly: scaling by a power of two commutes with every rounding."""
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_uniform(4096, 4096, 4096, BF16, 9)
    ad, bd = a.cuda(), b.cuda()
    c1 = torch.empty(4096, 4096, dtype=BF16, device="cuda")
    c2 = torch.empty_like(c1)
    capi.hgemm(c1, ad, bd)
    capi.hgemm(c2, ad * 2, bd)
    torch.cuda.synchronize()
    assert torch.equal(c1.float() * 2, c2.float())


def test_identity_b(cuda):
    """B = I: C must reproduce A bit for bit (each sum has one non-zero term)."""
    from peakgemm_b200 import capi

    a, _ = oracle.gemm_inputs_uniform(1000, 8, 2048, BF16, 10)
    eye = torch.eye(2048, dtype=BF16)
    c = helpers.garbage_like((1000, 2048), BF16, "cuda")
    capi.hgemm(c, a.cuda(), eye.cuda())
    torch.cuda.synchronize()
    assert torch.equal(c.cpu(), a)


def test_deterministic(cuda):
    from peakgemm_b200 import capi

    a, b = oracle.gemm_inputs_uniform(1024, 1024, 4096, F16, 11)
    ad, bd = a.cuda(), b.cuda()
    outs = []
    for _ in range(3):
        c = torch.empty(1024, 1024, dtype=F16, device="cuda")
        capi.hgemm(c, ad, bd)
        outs.append(c)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_roofline_probes(cuda):
    """The probes run and report plausible figures (tensor: between the reference kernel's and nominal peak)."""
    from peakgemm_b200 import capi

    tf, ms = capi.probe_tensor_peak(True, 2000)
    assert 500.0 < tf < 2600.0 and ms > 0
    src = torch.arange(1 << 22, dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    capi.probe_copy(dst, src)
    torch.cuda.synchronize()
    assert torch.equal(dst, src)
    assert capi.lib().pg_probe_tensor_peak(5, 10, None, None) == 1


# ---- tail split (pg_hgemm_ws): the last, partial wave of tiles cut into k-slices over the idle SM pairs
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("m,n,k", [
    (4096, 4096, 14336),    # 256 tiles on 74 pairs: remainder 34 -> 2 slices
    (1024, 14336, 8192),    # remainder 2 -> 4 slices
    (1024, 14336, 16384),   # remainder 2 -> 6 slices
    (1000, 14328, 8256),    # tails in m, n and k
])
def test_tail_split_matches_oracle_and_plain_kernel(cuda, m, n, k, dtype):
    from peakgemm_b200 import capi

    need = capi.hgemm_workspace_bytes(m, n, k)
    assert need > 0, "this shape is expected to qualify for the tail split on a 148-SM device"
    a, b = oracle.gemm_inputs_uniform(m, n, k, dtype, 15)
    ad, bd = a.cuda(), b.cuda()
    ws = torch.full((need,), 0xAB, dtype=torch.uint8, device="cuda")       # dirty on purpose
    split = helpers.garbage_like((m, n), dtype, "cuda")
    again = helpers.garbage_like((m, n), dtype, "cuda")
    plain = helpers.garbage_like((m, n), dtype, "cuda")
    small = helpers.garbage_like((m, n), dtype, "cuda")
    capi.hgemm_ws(split, ad, bd, ws)
    capi.hgemm_ws(again, ad, bd, ws)                 # same stream: the second call reuses the buffer after the first
    capi.hgemm(plain, ad, bd)
    capi.hgemm_ws(small, ad, bd, ws[:need // 2])     # too small: no split, same kernel as the plain call
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    helpers.check_gemm(split, a, b, exact_rows=False)
    assert torch.equal(split.view(torch.int16), again.view(torch.int16)), "tail split is not deterministic"
    assert torch.equal(small.view(torch.int16), plain.view(torch.int16))
    # only the remainder tiles may differ from the plain kernel, and only by fp32 summation order
    diff = (split.float() - plain.float()).abs()
    assert diff.max().item() <= 2.0 ** -6 * plain.float().abs().max().item()
    changed = (diff > 0).float().mean().item()
    # > 0: the split really ran (its tiles sum in another order); most of C, the whole tiles, is untouched
    assert 0.0 < changed < 0.2, changed


@pytest.mark.parametrize("m,n,k", [(512, 4096, 8192), (512, 4096, 14336), (300, 2056, 8200), (256, 8192, 8192),
                                   (512, 4096, 4096)])
def test_few_tiles_and_a_long_k_take_the_pair_split_k_kernel(cuda, m, n, k):
    """At most 40 tiles of 256 x 256 and k >= 4096: the automatic choice is two CTA pairs per tile sharing k through
    distributed shared memory (no workspace is asked for); same bits as the explicit variant, and deterministic."""
    from peakgemm_b200 import capi

    assert capi.hgemm_workspace_bytes(m, n, k) == 0
    a, b = oracle.gemm_inputs_uniform(m, n, k, BF16, 26)
    ad, bd = a.cuda(), b.cuda()
    auto = helpers.garbage_like((m, n), BF16, "cuda")
    again = helpers.garbage_like((m, n), BF16, "cuda")
    explicit = helpers.garbage_like((m, n), BF16, "cuda")
    plain = helpers.garbage_like((m, n), BF16, "cuda")
    capi.hgemm(auto, ad, bd)
    capi.hgemm_ws(again, ad, bd, None)
    capi.hgemm(explicit, ad, bd, variant=6)
    capi.hgemm(plain, ad, bd, variant=2, block_n=256)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    helpers.check_gemm(auto, a, b, exact_rows=False)
    assert torch.equal(auto.view(torch.int16), again.view(torch.int16))
    assert torch.equal(auto.view(torch.int16), explicit.view(torch.int16))
    assert not torch.equal(auto.view(torch.int16), plain.view(torch.int16)), "the k range was not split"


def test_tail_split_not_offered_where_it_cannot_help(cuda):
    from peakgemm_b200 import capi

    assert capi.hgemm_workspace_bytes(8192, 8192, 8192) == 0      # remainder 62 of 74: more than half a wave
    assert capi.hgemm_workspace_bytes(2048, 2048, 2048) == 0      # a single partial wave
    assert capi.hgemm_workspace_bytes(128, 4096, 4096) == 0       # small m: other kernels
    assert capi.hgemm_workspace_bytes(4096, 4096, 256) == 0       # k too short to slice
    assert capi.hgemm_workspace_bytes(1024, 14336, 4096) == 0     # 24 us tiles: reading the partial sums would cost the gain
    assert capi.hgemm_workspace_bytes(512, 4096, 4096) == 0       # the same for a problem of half a wave


def test_operator_uses_the_tail_split(cuda):
    import PeakGemm

    m, n, k = 1024, 14336, 8192
    assert torch.ops.PeakGemm.gemm_peak is not None
    a, b = oracle.gemm_inputs_llm(m, n, k, BF16, 16)
    c = helpers.garbage_like((m, n), BF16, "cuda")
    PeakGemm.gemm_peak(c, a.cuda(), b.cuda())
    torch.cuda.synchronize()
    helpers.check_gemm(c, a, b, exact_rows=False)


def test_tail_split_operator_is_capturable(cuda):
    """The operator on a shape that takes the tail split (scratch from torch's allocator, one memset, a cooperative
    launch) inside a CUDA graph: the replay on new inputs equals eager execution bit for bit."""
    import PeakGemm
    from peakgemm_b200 import capi

    m, n, k = 1024, 14336, 8192
    assert capi.hgemm_workspace_bytes(m, n, k) > 0
    a, b = oracle.gemm_inputs_llm(m, n, k, BF16, 17)
    ad, bd = a.cuda(), b.cuda()
    c = helpers.garbage_like((m, n), BF16, "cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        PeakGemm.gemm_peak(c, ad, bd)                 # per-device set-up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        PeakGemm.gemm_peak(c, ad, bd)
    a2, _ = oracle.gemm_inputs_llm(m, n, k, BF16, 18)
    ad.copy_(a2)
    c.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    replayed = c.clone()
    c.fill_(float("nan"))
    PeakGemm.gemm_peak(c, ad, bd)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.equal(replayed.view(torch.int16), c.view(torch.int16))
    helpers.check_gemm(c, a2, b, exact_rows=False)


def test_tail_split_on_two_streams_with_separate_workspaces(cuda):
    """Two split launches in flight on two streams, each with its own workspace (the documented way): both correct."""
    from peakgemm_b200 import capi

    m, n, k = 1024, 14336, 8192
    need = capi.hgemm_workspace_bytes(m, n, k)
    assert need > 0
    a, b = oracle.gemm_inputs_uniform(m, n, k, BF16, 19)
    ad, bd = a.cuda(), b.cuda()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    wss = [torch.empty(need, dtype=torch.uint8, device="cuda") for _ in streams]
    outs = [helpers.garbage_like((m, n), BF16, "cuda") for _ in streams]
    torch.cuda.synchronize()
    for rep in range(3):
        for s, ws, o in zip(streams, wss, outs):
            with torch.cuda.stream(s):
                capi.hgemm_ws(o, ad, bd, ws, stream=s)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    helpers.check_gemm(outs[0], a, b, exact_rows=False)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_synchronised_producers_on_two_streams(cuda):
    """Two large GEMMs in flight on two streams.  Each takes the 512 x 256 kernel whose producers meet at a counter;
    with two persistent grids competing for the SMs part of a grid is not resident while the rest already waits at
    a meeting point.  A wait there has a short patience and no consequence for the result: both launches must finish
    without a status code and give the bits of a launch that ran alone."""
    from peakgemm_b200 import capi

    m, n, k = 8192, 8192, 2048
    assert capi.hgemm_config(m, n, k) == (5, 256)
    a, b = oracle.gemm_inputs_uniform(m, n, k, BF16, 23)
    ad, bd = a.cuda(), b.cuda()
    alone = helpers.garbage_like((m, n), BF16, "cuda")
    capi.hgemm(alone, ad, bd)
    torch.cuda.synchronize()
    rows = torch.arange(32) * 256 + 9
    helpers.check_gemm(alone[rows.cuda()], a[rows], b, exact_rows=False)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [helpers.garbage_like((m, n), BF16, "cuda") for _ in streams]
    torch.cuda.synchronize()
    for _ in range(4):
        for s, o in zip(streams, outs):
            with torch.cuda.stream(s):
                capi.hgemm(o, ad, bd, stream=s)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    for o in outs:
        assert torch.equal(o.view(torch.int16), alone.view(torch.int16))

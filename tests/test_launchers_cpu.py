"""Host-side argument checks of the native launchers.

Every launcher validates shapes, alignment and the collective-coupling parameters before it
touches the device and returns a small error code instead of launching; a wrong shard size or a
misaligned slab must never reach a kernel that stores into a peer's memory.  These checks run
without a GPU: the library is loaded and the launchers are called with arguments that must be
refused (no pointer is dereferenced on the refusing paths).
"""
import ctypes

import pytest

VP, I, LL, F, D = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double
PTR = 4096          # an aligned, never dereferenced address


@pytest.fixture(scope="module")
def lib():
    try:
        from kotodama_b200.ops import _build
        return _build.load()
    except Exception as e:                                   # no compiler and no built library
        pytest.skip(f"native library unavailable: {e}")


def _ag(lib, M, K, rows, dim, own, flags=True):
    fl = (ctypes.c_int * 8)() if flags else None
    return lib.kb_gemm_2cta_ag(VP(PTR), VP(PTR), VP(PTR), VP(None), I(M), I(256), I(K), LL(K), LL(K), LL(256),
                               I(0), I(0), F(1.0), F(0.0), fl, I(1), I(rows), I(dim), I(own), D(1.0), VP(None),
                               VP(None))


def test_all_gather_gemm_refuses_bad_shards(lib):
    assert _ag(lib, 1024, 256, 512, 0, 0, flags=False) == 5          # no flag array
    assert _ag(lib, 1024, 256, 128, 0, 0) == 5                       # shard is not whole 256-row tiles
    assert _ag(lib, 1024, 256, 96, 1, 0) == 5                        # K shard is not whole 64-wide k-blocks
    assert _ag(lib, 1024, 256, 512, 0, 8) == 5                       # rank out of range
    assert _ag(lib, 1024, 256, 512, 0, 2) == 5                       # rank's shard lies beyond M
    assert _ag(lib, 1280, 256, 512, 0, 0) == 5                       # M is not a whole number of shards
    assert _ag(lib, 8192, 256, 256, 0, 0) == 5                       # more than eight shards


def _rs(lib, M, N, rows, world, rank, slabs=None, ldc=None):
    arr = lambda v: (VP * 8)(*(list(v) + [None] * (8 - len(v))))
    slabs = slabs if slabs is not None else [PTR] * world
    return lib.kb_gemm_2cta_rs(VP(PTR), VP(PTR), I(M), I(N), I(64), LL(64), LL(64), LL(ldc or N), I(0), I(0),
                               F(1.0), arr(slabs), arr([PTR] * world), I(world), I(rank), I(rows), VP(None),
                               VP(None))


def test_gemm_reduce_scatter_refuses_bad_slabs(lib):
    assert _rs(lib, 1024, 256, 128, 8, 0) == 5                       # slab rows are not whole 256-row tiles
    assert _rs(lib, 1024, 256, 256, 2, 0) == 5                       # M != world * rows
    assert _rs(lib, 512, 256, 256, 2, 2) == 5                        # rank out of range
    assert _rs(lib, 512, 252, 256, 2, 0) == 6                        # row segments would not be 16-byte pieces
    assert _rs(lib, 512, 256, 256, 2, 0, ldc=260) == 6
    assert _rs(lib, 512, 256, 256, 2, 0, slabs=[PTR, None]) == 6     # a peer slab is missing
    assert _rs(lib, 512, 256, 256, 2, 0, slabs=[PTR, PTR + 8]) == 6  # or misaligned


def test_arrival_counts(lib):
    # narrow (256-column) tiles: every 128-row block of a slab, tile column and epilogue warp arrives once
    assert lib.kb_gemm_2cta_rs_arrivals(I(4096), I(3072), I(2048)) == (2048 // 128) * (3072 // 256) * 4
    assert lib.kb_gemm_2cta_rs_arrivals(I(512), I(300), I(256)) == 2 * 2 * 4
    # 1-CTA kernel: 128 x 256 tiles
    assert lib.kb_gemm_rs_arrivals(I(3072), I(2048)) == (2048 // 128) * (3072 // 256) * 4


def test_quantisers_refuse_ragged_shapes(lib):
    assert lib.kb_quant_rows(VP(PTR), LL(200), VP(PTR), LL(200), VP(PTR), I(4), I(200), I(0), VP(None)) == 5      # K % 128
    assert lib.kb_quant_blocks(VP(PTR), LL(256), VP(PTR), VP(PTR), VP(None), VP(None), I(100), I(256), I(0), VP(None)) == 5
    assert lib.kb_quant_cols_t(VP(PTR), LL(256), VP(PTR), VP(PTR), I(100), I(256), I(0), VP(None)) == 5           # M % 128


def _skinny(lib, M=64, N=3072, K=3072, lda=None, ldb=None, a=PTR, b=PTR, bn=0, flags=0):
    return lib.kb_gemm_skinny(VP(a), VP(b), VP(PTR), VP(None), I(M), I(N), I(K), LL(lda if lda is not None else K),
                              LL(ldb if ldb is not None else K), LL(N), LL(0), F(1.0), F(0.0), I(0), I(bn), I(flags), VP(None), VP(None))


def test_decode_size_gemm_refuses_bad_arguments(lib):
    assert _skinny(lib, M=0) == 5 and _skinny(lib, M=129) == 5 and _skinny(lib, N=0) == 5 and _skinny(lib, K=0) == 5
    assert _skinny(lib, lda=3076) == 6                               # row stride of A is not a multiple of 8 elements
    assert _skinny(lib, ldb=3076) == 6
    assert _skinny(lib, a=PTR + 2) == 6 and _skinny(lib, b=PTR + 8) == 6     # operands must be 16-byte aligned for TMA
    assert _skinny(lib, bn=64) == 5                                  # tile widths are 128 or 256
    assert _skinny(lib, K=3100, flags=1) == 6                        # the tile-major weight copy needs whole 64-deep k-blocks


def _skinny_ar(lib, M=64, N=3072, world=2, rank=0, slot=64 * 3072, recv=None, flags=None, out=PTR, epoch=PTR, counters=PTR):
    arr = lambda v: (VP * 8)(*(list(v) + [None] * (8 - len(v))))
    recv = recv if recv is not None else [PTR] * max(world, 0)
    flags = flags if flags is not None else [PTR] * max(world, 0)
    return lib.kb_gemm_skinny_allreduce(VP(PTR), VP(PTR), VP(out), VP(None), I(M), I(N), I(1024), LL(1024), LL(1024), I(0), arr(recv),
                                        arr(flags), I(world), I(rank), LL(slot), VP(epoch), VP(counters), D(1.0), VP(None), VP(None))


def test_fused_gemm_allreduce_refuses_bad_arguments(lib):
    assert _skinny_ar(lib, world=0) == 5 and _skinny_ar(lib, world=9, recv=[PTR] * 8, flags=[PTR] * 8) == 5
    assert _skinny_ar(lib, rank=2) == 5 and _skinny_ar(lib, rank=-1) == 5
    assert _skinny_ar(lib, N=3076) == 5                              # rows are pushed as 16-byte pieces
    assert _skinny_ar(lib, slot=1000) == 5                           # M * N does not fit a receive slot
    assert _skinny_ar(lib, epoch=None) == 5 and _skinny_ar(lib, counters=None) == 5
    assert _skinny_ar(lib, recv=[PTR, None]) == 6 and _skinny_ar(lib, flags=[None, PTR]) == 6      # a peer buffer is missing
    assert _skinny_ar(lib, recv=[PTR, PTR + 4]) == 6 and _skinny_ar(lib, out=PTR + 8) == 6         # or misaligned


def test_serving_kernels_refuse_bad_arguments(lib):
    qk = lambda hd=128, kp=PTR, vp=PTR, slot=PTR: lib.kb_qknorm_rope_append(
        VP(PTR), VP(PTR), VP(PTR), VP(PTR), VP(PTR), VP(PTR), VP(PTR), I(4), I(4), I(24), I(8), I(hd), I(0), F(1e-5), VP(None),
        VP(kp), VP(vp), VP(slot), LL(1024), VP(None), VP(None))
    assert qk(kp=None) == 5 and qk(vp=None) == 5 and qk(slot=None) == 5       # the append needs pages and slots
    assert qk(hd=96) == 5                                                     # head sizes 64 and 128
    dec = lambda n_q=24, n_kv=8, split=512: lib.kb_paged_decode_merged(
        VP(PTR), LL(3072), VP(PTR), VP(PTR), VP(PTR), I(80), VP(PTR), I(4), I(n_q), I(n_kv), I(128), I(1024), I(split), F(0.088),
        VP(PTR), VP(PTR), VP(PTR), LL(3072), I(64), VP(PTR), VP(None))
    assert dec(n_q=25) == 5 and dec(split=500) == 5 and dec(split=4096) == 5  # whole head groups, whole pages, at most 2048 tokens per split
    assert lib.kb_kv_append(VP(PTR), VP(PTR), LL(1024), LL(1024), VP(PTR), VP(PTR), VP(PTR), I(4), I(1020), I(128), LL(1024), VP(None),
                            VP(None)) == 5                                    # rows are copied as 16-byte pieces
    assert lib.kb_swiglu_fwd(VP(PTR), VP(PTR), LL(4), I(8188), VP(None)) == 5
    assert lib.kb_pack_weight_tiles(VP(PTR), LL(3100), VP(PTR), I(3072), I(3100), VP(None)) == 5

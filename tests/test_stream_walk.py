"""The prompt-shaped product's stream walk, on the host: the K blocks of all tiles in a row, cut into one range per
CTA.  The kernel's waits are safe because of what is checked here: a CTA leaves at most one part, as its first
piece; an owner's tile is its last piece; a part's owner is the nearest CTA before it that holds the tile's
first K block; every K block of every tile belongs to exactly one piece."""
import ctypes

import pytest

from picolm_b200.ops._lib import _fn

WHOLE, PART, OWNER = 0, 1, 2


def pieces(tiles, n_kb, ctas, cta):
    buf = (ctypes.c_int * (4 * 64))()
    n = _fn("gemm_tc_wide", "plm_gemm_tc_wide_pieces")(tiles, n_kb, ctas, cta, ctypes.cast(buf, ctypes.c_void_p), 64)
    assert n <= 64
    return [tuple(buf[4 * i:4 * i + 4]) for i in range(n)]


@pytest.mark.parametrize("tiles,n_kb,ctas", [(128, 128, 148), (192, 32, 148), (128, 32, 148), (8, 64, 64), (1, 40, 5),
                                             (3, 7, 2), (149, 1, 148), (1792, 224, 148), (5, 1000, 148), (16, 32, 64),
                                             (147, 33, 148), (296, 5, 148), (2, 9, 18)])
def test_every_k_block_once_and_waits_without_cycles(tiles, n_kb, ctas):
    seen = {}
    for cta in range(ctas):
        ps = pieces(tiles, n_kb, ctas, cta)
        for i, (tile, b, e, kind) in enumerate(ps):
            assert 0 <= tile < tiles and 0 <= b < e <= n_kb
            assert kind == (PART if b > 0 else OWNER if e < n_kb else WHOLE)
            if kind == PART:
                assert i == 0                                   # a part is its CTA's first piece: it waits for nothing
            if kind == OWNER:
                assert i == len(ps) - 1                         # an owner's tile is its CTA's last piece
            for kb in range(b, e):
                assert (tile, kb) not in seen
                seen[(tile, kb)] = cta
    assert len(seen) == tiles * n_kb
    # the parts of a tile come from the CTAs right after its owner, one each, in the order of K
    for tile in range(tiles):
        ctas_of = []
        for kb in range(n_kb):
            if not ctas_of or ctas_of[-1] != seen[(tile, kb)]:
                ctas_of.append(seen[(tile, kb)])
        assert ctas_of == list(range(ctas_of[0], ctas_of[0] + len(ctas_of)))


def test_when_the_stream_walk_is_taken():
    how = _fn("gemm_tc_wide", "plm_gemm_tc_wide_how")
    out = (ctypes.c_int * 3)()

    def ask(T, F, K, epilogue, slots):
        assert how(T, F, K, epilogue, slots, ctypes.cast(out, ctypes.c_void_p)) == 0
        return tuple(out)

    assert ask(4096, 2048, 8192, 0, 148)[2] == 0                # 256 tiles, 1.73 rounds: whole tiles (measured faster)
    assert ask(1536, 2048, 8192, 0, 148)[2] == 148              # 96 tiles: a third of the SMs would idle
    assert ask(1536, 2048, 8192, 0, 0)[2] == 0                  # no workspace: whole tiles
    assert ask(128 * 148, 256 * 4, 512, 0, 148)[2] == 0         # four full rounds: whole tiles
    assert ask(2048, 2048, 8192, 0, 148)[2] == 0                # 128 tiles for 148 SMs: the parts would cost more
    assert ask(1024, 2048, 8192, 0, 148)[2] == 128              # 64 tiles: less than half of the SMs would work; two CTAs a tile
    bn, splits, streamed = ask(128, 2048, 2048, 0, 148)
    assert splits > 1 and streamed == 0                         # few tiles, store: K in parts through scratch memory
    assert ask(128, 2048, 2048, 2, 148)[1] == 1                 # the other epilogues never cut K that way
    assert ask(1024, 2048, 8192, 2, 100)[2] == 100              # no more CTAs than slots


def test_which_form_a_shape_takes():
    """The dispatcher's choice between pairs of CTAs and single CTAs (decided on the host, from the shape alone)."""
    from picolm_b200.ops.gemm import pair_pays
    assert pair_pays(2048, 2048, 8192, 2) and pair_pays(2048, 16384, 2048, 1) and pair_pays(2048, 3072, 2048, 0)
    assert not pair_pays(2048, 2048, 8200, 2)                   # K no multiple of 64: the pairs' copies take whole tiles
    assert not pair_pays(200, 2048, 2048, 0)                    # fewer than 256 tokens
    assert not pair_pays(2048, 200, 2048, 0)                    # fewer than 256 features
    assert pair_pays(1024, 2048, 8192, 2)                       # 32 tiles with a long K: the pairs walk them as a stream
    assert not pair_pays(1024, 2048, 2048, 2)                   # 32 tiles with a short K: nothing to share out
    assert not pair_pays(512, 2048, 8192, 0)                    # few tiles, store: single CTAs cut K through scratch memory

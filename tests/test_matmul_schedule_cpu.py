"""The persistent MatMul kernel's schedule (rmlk_b200_matmul_schedule), checked on the host: the ranges the CTAs take
cover every k-block of every tile exactly once, a tile is shared by at most 16 consecutive CTAs, every CTA has at most
two partial tiles (its first and its last), and the slot / flag addressing that the kernel derives from the same
arithmetic gives every partial tile its own slot and every (writer, reader) pair its own flag."""
import ctypes

import pytest

SHAPES = [(64, 16384, 2048), (64, 3072, 2048), (64, 2048, 2048), (64, 2048, 8192), (64, 128256, 2048), (64, 8192, 2048), (17, 128, 32),
          (33, 256, 64), (64, 14336, 4096), (64, 4096, 14336), (4096, 8192, 2048), (4096, 14336, 4096), (4096, 4096, 14336), (100, 384, 96),
          (200, 256, 512), (300, 128, 2048), (65, 128, 4096), (64, 18944, 2048), (24, 128, 32 * 500), (64, 148 * 128, 64), (130, 2688, 1024)]
MAX_GROUP = 16


def schedule(m, n, k):
    from rmlk_b200._lib import lib
    out = (ctypes.c_int64 * 8)()
    rc = lib().rmlk_b200_matmul_schedule(ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k), out)
    assert rc == 0
    return dict(zip(["mt", "k_iters", "m_tiles", "gran", "ctas", "tiles", "units", "ws_bytes"], list(out)))


@pytest.mark.parametrize("shape", SHAPES)
def test_schedule_covers_every_k_block_once(shape):
    m, n, k = shape
    s = schedule(m, n, k)
    K, G, U, gran = s["k_iters"], s["ctas"], s["units"], s["gran"]
    assert s["mt"] == (64 if m <= 64 else 128) and K == k // 32 and s["tiles"] == (n // 128) * s["m_tiles"]
    assert U * gran == s["tiles"] * K and 1 <= G <= 148 and G <= U

    def owner(x):  # the kernel's formula for the CTA that owns linear k-block x (gran == 1)
        return ((x + 1) * G - 1) // U

    def slot_of(c, tile):
        first_tile = (U * c // G) // K
        return 2 * c + (0 if first_tile == tile else 1)

    covered = {}
    slots, flags_written, flags_read = {}, set(), set()
    for c in range(G):
        a, b = (U * c // G) * gran, (U * (c + 1) // G) * gran
        assert b > a
        pos, partial_tiles = a, []
        while pos < b:
            tile, kb0 = divmod(pos, K)
            ln = min(K - kb0, b - pos)
            covered.setdefault(tile, []).append((kb0, kb0 + ln, c))
            if not (kb0 == 0 and ln == K):
                assert gran == 1
                partial_tiles.append(tile)
                g0, g1 = owner(tile * K), owner(tile * K + K - 1)
                assert g0 <= c <= g1 and g1 - g0 + 1 <= MAX_GROUP
                sl = slot_of(c, tile)
                assert sl not in slots
                slots[sl] = (c, tile)
                for reader in range(g1 - g0 + 1):
                    flags_written.add((sl, reader))
                rank = c - g0
                for member in range(g0, g1 + 1):
                    flags_read.add((slot_of(member, tile), rank))
            pos += ln
        assert len(partial_tiles) <= 2 and len(set(partial_tiles)) == len(partial_tiles)
    for tile in range(s["tiles"]):
        segs = sorted(covered[tile])
        assert segs[0][0] == 0 and segs[-1][1] == K
        for (a0, a1, c0), (b0, b1, c1) in zip(segs, segs[1:]):
            assert a1 == b0 and c1 == c0 + 1          # consecutive CTAs, no gap, no overlap
    assert flags_read == flags_written                # every awaited flag is raised by somebody, and nothing else is raised
    need = 0
    if slots:
        flag_bytes = (2 * G * MAX_GROUP * 8 + 255) // 256 * 256
        need = flag_bytes + 2 * G * s["mt"] * 128 * 4
        assert max(slots) < 2 * G
    assert s["ws_bytes"] == need

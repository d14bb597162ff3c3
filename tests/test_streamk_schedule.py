"""Model of the stream-K work split of the token-tile GEMM (csrc/gemm/gemm_bf16_sm100.cu: TokSched and the partial-tile
protocol), in the kernel's own integer arithmetic.

Checked for many (tiles, K blocks, unit size, grid) combinations: every (tile, K block) is computed exactly once; a CTA
has at most one partial tile per scratch slot; and the CTA that sums a tile's partial results finds, from the tile index
alone, exactly the CTAs and slots that the writers used, in the order of their K ranges.
"""
import random


def cta_pieces(c, G, num_tiles, num_kb, kgroup):
    num_kg = -(-num_kb // kgroup)
    U = num_tiles * num_kg
    u_begin, u_end = U * c // G, U * (c + 1) // G
    u, out = u_begin, []
    while u < u_end:
        t = u // num_kg
        a = t * num_kg
        e = min(u_end, a + num_kg)
        kb0, kb1 = (u - a) * kgroup, min(num_kb, (e - a) * kgroup)
        whole = kb0 == 0 and kb1 == num_kb
        slot = None if whole else (0 if u == u_begin else 1)
        out.append((t, kb0, kb1, slot))
        u = e
    return out


def reader_view(t, G, num_tiles, num_kb, kgroup):
    num_kg = -(-num_kb // kgroup)
    U = num_tiles * num_kg
    a = t * num_kg
    c0 = ((a + 1) * G + U - 1) // U - 1
    n = ((a + num_kg) * G + U - 1) // U - c0
    return [(c, 0 if U * c // G >= a else 1) for c in range(c0, c0 + n)]


def test_every_k_block_once_and_reader_finds_the_writers():
    rng = random.Random(0)
    cases = [(48, 64, 4, 148), (32, 192, 4, 148), (192, 64, 4, 148), (5, 80, 2, 148), (1, 64, 1, 64), (3, 7, 2, 5), (24, 64, 4, 148)]
    for _ in range(300):
        tiles, num_kb, kg = rng.randint(1, 300), rng.randint(1, 200), rng.choice([1, 2, 3, 4, 8])
        kg = min(kg, num_kb)
        U = tiles * -(-num_kb // kg)
        cases.append((tiles, num_kb, kg, min(rng.randint(1, 160), U)))
    for tiles, num_kb, kg, G in cases:
        G = min(G, tiles * -(-num_kb // kg))
        seen = {}
        writers = {}
        for c in range(G):
            pieces = cta_pieces(c, G, tiles, num_kb, kg)
            assert pieces, "a CTA without work would be counted by a reader and never arrive"
            slots = [p[3] for p in pieces if p[3] is not None]
            assert len(slots) == len(set(slots)), "two partial tiles of one CTA in the same slot"
            for t, kb0, kb1, slot in pieces:
                assert kb0 < kb1
                for kb in range(kb0, kb1):
                    assert (t, kb) not in seen
                    seen[(t, kb)] = c
                if slot is not None:
                    writers.setdefault(t, []).append((kb0, c, slot))
        assert len(seen) == tiles * num_kb
        for t, w in writers.items():
            assert len(w) >= 2, "a partial tile has at least two contributors"
            assert [(c, s) for _, c, s in sorted(w)] == reader_view(t, G, tiles, num_kb, kg)


def finish_kernel_writes(M, N, block_n, pair, raster_group):
    """(row, column) pairs written by gemm_splitk_finish_kernel's grid, in the kernel's index arithmetic: grid
    (blocks of 32 live rows, 128-column parts of a tile, tiles), block = 8 warps x 32 lanes; in the write phase warp w
    handles rows 4w .. 4w + 3 of the block and lane l the four columns 4l .. 4l + 3 of the part."""
    tile_rows = 256 if pair else 128
    m_tiles, n_tiles = -(-M // tile_rows), -(-N // block_n)
    live_rows = min(M, tile_rows)
    out = []
    for t in range(m_tiles * n_tiles):
        per_group = raster_group * n_tiles
        g = t // per_group
        first = g * raster_group
        gm = min(raster_group, m_tiles - first)
        within = t - g * per_group
        mt, nt = first + within % gm, within // gm
        for bx in range(-(-live_rows // 32)):
            row0 = mt * tile_rows + bx * 32
            if row0 >= M:
                continue
            for by in range(-(-block_n // 128)):
                c0 = nt * block_n + by * 128
                for warp in range(8):
                    for rr in range(4):
                        r = row0 + warp * 4 + rr
                        for lane in range(32):
                            c = c0 + lane * 4
                            if r < M and by * 128 + lane * 4 < block_n and c < N:
                                out.extend((r, c + j) for j in range(4) if c + j < N)
    return out


def test_reduce_kernel_grid_covers_every_output_element_once():
    for M, N, block_n, pair, grp in [(256, 4096, 256, 1, 8), (200, 1000, 256, 1, 8), (64, 6144, 256, 0, 16), (130, 3200, 128, 0, 16),
                                     (300, 1100, 256, 1, 8), (7, 136, 128, 0, 16), (512, 640, 128, 1, 8)]:
        w = finish_kernel_writes(M, N, block_n, pair, grp)
        assert len(w) == len(set(w)) == M * N, (M, N, block_n, pair)

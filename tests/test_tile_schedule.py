"""Host-side checks of the arithmetic the step kernel uses to hand out tiles (cudarl-arena_b200/csrc/tile_engine.cu, the tile loop
of k_tile_step): the queue layout must cover every tile exactly once whatever the numbers of tiles, SMs and blocks and whichever way
a step walks its queues, and the reciprocal multiplication must split a tile index into row and column exactly."""
import random


def tiles_of_queue(ntiles, nq_sms, grid_blocks, queue, flip):
    """Tiles a queue hands out, in ticket order: the kernel's `ticket_tile` for tickets 0 .. qn - 1."""
    qn_total = min(nq_sms, grid_blocks)
    qn = ntiles // qn_total + (1 if queue < ntiles % qn_total else 0)
    return [queue + qn_total * ((qn - 1 - t) if flip else t) for t in range(qn)]


def test_queues_cover_every_tile_exactly_once():
    rng = random.Random(5)
    cases = [(65536, 148, 1036), (64, 148, 16), (1, 148, 1), (147, 148, 37), (148, 148, 37), (149, 148, 38), (16384, 148, 888), (999, 132, 250)]
    cases += [(rng.randrange(1, 5000), rng.choice([1, 7, 108, 132, 148]), rng.randrange(1, 1200)) for _ in range(60)]
    for ntiles, sms, blocks in cases:
        grid = min(blocks, (ntiles + 3) // 4)              # the launch never has more blocks than tiles / warps per block
        nq = min(sms, grid)
        for flip in (False, True):
            seen = []
            for q in range(nq):                            # every queue is served by the blocks q, q + nq, ... of the launch
                assert q < grid
                seen += tiles_of_queue(ntiles, sms, grid, q, flip)
            assert sorted(seen) == list(range(ntiles)), (ntiles, sms, blocks, flip)


def test_reciprocal_split_of_a_tile_index():
    rng = random.Random(9)
    for d in [1, 2, 3, 5, 7, 13, 64, 148, 255, 256, 257, 1000, 4096, 65535, 65536, 1 << 20]:
        rcp = ((1 << 32) // d) if d > 1 else 0xFFFFFFFF    # tp.tiles_x_rcp
        for n in [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, (1 << 24) - 1, (1 << 32) - 1] + [rng.randrange(1 << 32) for _ in range(500)]:
            if not 0 <= n < (1 << 32):
                continue
            q = (n * rcp) >> 32                            # __umulhi(n, rcp)
            r = n - q * d
            if r >= d:                                     # the kernel's single correction
                q, r = q + 1, r - d
            assert (q, r) == divmod(n, d), (n, d)

"""Byte layout of the N-sharded prefill MLP block's peer buffer (qwen35x_b200/sharding.py:MlpLayout): no GPU needed."""
import numpy as np


def test_layout_regions_cover_the_intermediate_exactly():
    """The regions of all shards tile the code bytes and the scale tiles of h without gap or overlap."""
    from qwen35x_b200 import sharding

    for world, m, hidden, inter in ((8, 4096, 2560, 9216), (3, 130, 256, 384), (2, 64, 128, 64)):
        L = sharding.MlpLayout(m, hidden, inter)
        seen = np.zeros(L.total, dtype=np.int32)
        for (b, c) in sharding.shard_layout(2 * inter, world):
            for off, rows, rb, ld in L.h_regions(b // 2, c // 2):
                for r in range(rows):
                    seen[off + r * ld: off + r * ld + rb] += 1
        assert np.all(seen[L.codes_off:L.codes_off + m * L.codes_ld] == 1)
        assert np.all(seen[L.scales_off:L.scales_off + L.scales_bytes] == 1)
        assert seen[L.out_off:].sum() == 0

"""`@dt.kernel` matmul of examples/deuteron/01_matmul.py:12-18 of the reference."""

import newt_b200.deuteron as dt


@dt.kernel
def tile_matmul(x, y, out):
    for tile_m, tile_n in dt.tile([x.shape[0], y.shape[1]]):
        acc = dt.zeros([tile_m, tile_n], dtype=dt.float32)
        for tile_k in dt.tile(x.shape[1]):
            acc += x[tile_m, tile_k] @ y[tile_k, tile_n]
        out[tile_m, tile_n] = acc

"""Plain numpy statement of the expert-parallel dispatch / combine protocol (test infrastructure):
what `shrike_ep_encode_dispatch` and `shrike_ep_encode_combine` must compute."""
import numpy as np

INVALID = 0xFFFFFFFF


def pack(x, ids, w, world, experts_per_rank, cap):
    T, K = ids.shape
    d = x.shape[1]
    send_x = np.zeros((world, cap, d), dtype=x.dtype)
    send_ids = np.full((world, cap, K), INVALID, dtype=np.uint32)
    send_w = np.zeros((world, cap, K), dtype=np.float32)
    counts = np.zeros(world, dtype=np.uint32)
    row_of = np.full((T, world), -1, dtype=np.int32)
    for t in range(T):
        for g in range(world):
            here = (ids[t] // experts_per_rank) == g
            if here.any():
                r = counts[g]
                counts[g] += 1
                row_of[t, g] = r
                send_x[g, r] = x[t]
                send_ids[g, r] = np.where(here, ids[t] - g * experts_per_rank, INVALID)
                send_w[g, r] = np.where(here, w[t], 0)
    return send_x, send_ids, send_w, counts, row_of


def combine(recv_y, row_of, y_home):
    T, world = row_of.shape
    y = np.zeros((T, recv_y.shape[2]), dtype=np.float32) if y_home is None else y_home.astype(np.float32).copy()
    for t in range(T):
        for g in range(world):
            if row_of[t, g] >= 0:
                y[t] += recv_y[g, row_of[t, g]]
    return y

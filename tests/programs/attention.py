"""Single-head attention written as a tt-lang tile program with the block operators and reductions
(`ttl.math.reduce_max / reduce_sum`, docs/sphinx/specs/TTLangSpecification.md:750-755): per strip of 32 queries,
S = Q @ K^T (K given transposed), P = softmax(scale * S + mask) along the keys, O = P @ V.  The reference has no
attention example; this is the plain (score-matrix) form, not the blocked online-softmax form of the fused
attention kernel."""
# type: ignore
import math

import ttl
import ttnn  # noqa: F401

N_CORES = 4


@ttl.kernel(grid=(2, 2))
def attention_rows(q, kt, v, mask, scale, one, out):
    """q [S, D], kt [D, S], v [S, D], mask [S, S] (added to the scaled scores), scale / one: [32, 32] tiles whose
    element [0, 0] is the softmax scale / 1.0, out [S, D]; all bfloat16 or all float32."""
    st, dt = q.shape[0] // 32, q.shape[1] // 32
    per_core = math.ceil(st / N_CORES)
    q_cb = ttl.make_circular_buffer_like(q, shape=(1, dt), buffer_factor=2)
    kt_cb = ttl.make_circular_buffer_like(kt, shape=(dt, st), buffer_factor=2)
    v_cb = ttl.make_circular_buffer_like(v, shape=(st, dt), buffer_factor=2)
    mask_cb = ttl.make_circular_buffer_like(mask, shape=(1, st), buffer_factor=2)
    scale_cb = ttl.make_circular_buffer_like(scale, shape=(1, 1), buffer_factor=2)
    one_cb = ttl.make_circular_buffer_like(one, shape=(1, 1), buffer_factor=2)
    s_cb = ttl.make_circular_buffer_like(mask, shape=(1, st), buffer_factor=2)
    m_cb = ttl.make_circular_buffer_like(q, shape=(1, 1), buffer_factor=2)
    e_cb = ttl.make_circular_buffer_like(mask, shape=(1, st), buffer_factor=2)
    d_cb = ttl.make_circular_buffer_like(q, shape=(1, 1), buffer_factor=2)
    out_cb = ttl.make_circular_buffer_like(out, shape=(1, dt), buffer_factor=2)

    def my_rows():
        core = ttl.core(dims=1)
        return range(core * per_core, min((core + 1) * per_core, st))

    @ttl.compute()
    def compute():
        for _r in my_rows():
            with (q_cb.wait() as qb, kt_cb.wait() as ktb, v_cb.wait() as vb, mask_cb.wait() as mb,
                  scale_cb.wait() as cb, one_cb.wait() as ob):
                with s_cb.reserve() as sb:
                    sb.store(qb @ ktb)                                           # (1, D) @ (D, S) -> (1, S)
                with s_cb.wait() as sb, e_cb.reserve() as zb:
                    zb.store(sb * ttl.math.broadcast(cb, dims=[0, 1]) + mb)      # scaled, masked scores
                with e_cb.wait() as zb:
                    with m_cb.reserve() as mx:
                        mx.store(ttl.math.reduce_max(zb, ob, dims=[1]))
                    with m_cb.wait() as mx, e_cb.reserve() as eb:
                        eb.store(ttl.math.exp(zb - ttl.math.broadcast(mx, dims=[1])))
                with e_cb.wait() as eb:
                    with d_cb.reserve() as db:
                        db.store(ttl.math.reduce_sum(eb, ob, dims=[1]))
                    with d_cb.wait() as db, out_cb.reserve() as yb:
                        yb.store((eb / ttl.math.broadcast(db, dims=[1])) @ vb)   # (1, S) @ (S, D) -> (1, D)

    @ttl.datamovement()
    def dm0():
        for r in my_rows():
            for cb_, src in ((q_cb, q[r:r + 1, 0:dt]), (kt_cb, kt[0:dt, 0:st]), (v_cb, v[0:st, 0:dt]),
                             (mask_cb, mask[r:r + 1, 0:st]), (scale_cb, scale[0:1, 0:1]), (one_cb, one[0:1, 0:1])):
                with cb_.reserve() as blk:
                    tx = ttl.copy(src, blk)
                    tx.wait()

    @ttl.datamovement()
    def dm1():
        for r in my_rows():
            with out_cb.wait() as yb:
                tx = ttl.copy(yb, out[r:r + 1, 0:dt])
                tx.wait()


# --------------------------------------------------------------------------------------------------------------
# The same attention as THREE kernels that the reference simulator can run at any head dimension: its block matmul
# multiplies (1,1) @ (1,1) tile blocks and accumulates over K with store(acc=True) (python/sim/block.py:805-920),
# so the scores and the probabilities travel through tensors instead of circular buffers.
# --------------------------------------------------------------------------------------------------------------
@ttl.kernel(grid=(2, 2))
def tile_matmul(a, b, out):
    """out = a @ b in 1x1-tile blocks, K accumulated with store(acc=True); output tiles dealt round-robin to the cores."""
    mt, kt_, nt = a.shape[0] // 32, a.shape[1] // 32, b.shape[1] // 32
    a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
    o_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

    def my_tiles():
        return list(range(mt * nt))[ttl.core(dims=1)::N_CORES]

    @ttl.compute()
    def mm():
        for _ in my_tiles():
            with o_cb.reserve() as ob:
                for _k in range(kt_):
                    with a_cb.wait() as ab, b_cb.wait() as bb:
                        ob.store(ab @ bb, acc=True)

    @ttl.datamovement()
    def rd():
        for t in my_tiles():
            for k in range(kt_):
                with a_cb.reserve() as ab, b_cb.reserve() as bb:
                    ta = ttl.copy(a[t // nt, k], ab)
                    tb = ttl.copy(b[k, t % nt], bb)
                    ta.wait()
                    tb.wait()

    @ttl.datamovement()
    def wr():
        for t in my_tiles():
            with o_cb.wait() as ob:
                tx = ttl.copy(ob, out[t // nt, t % nt])
                tx.wait()


@ttl.kernel(grid=(2, 2))
def masked_softmax_rows(s, mask, scale, one, p):
    """p = softmax(scale * s + mask) along each row, one strip of 32 rows per step."""
    rt, ct = s.shape[0] // 32, s.shape[1] // 32
    per_core = math.ceil(rt / N_CORES)
    s_cb = ttl.make_circular_buffer_like(s, shape=(1, ct), buffer_factor=2)
    mask_cb = ttl.make_circular_buffer_like(mask, shape=(1, ct), buffer_factor=2)
    scale_cb = ttl.make_circular_buffer_like(scale, shape=(1, 1), buffer_factor=2)
    one_cb = ttl.make_circular_buffer_like(one, shape=(1, 1), buffer_factor=2)
    z_cb = ttl.make_circular_buffer_like(s, shape=(1, ct), buffer_factor=2)
    m_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
    d_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
    p_cb = ttl.make_circular_buffer_like(p, shape=(1, ct), buffer_factor=2)

    def my_rows():
        core = ttl.core(dims=1)
        return range(core * per_core, min((core + 1) * per_core, rt))

    @ttl.compute()
    def compute():
        for _r in my_rows():
            with s_cb.wait() as sb, mask_cb.wait() as mb, scale_cb.wait() as cb, one_cb.wait() as ob:
                with z_cb.reserve() as zb:
                    zb.store(sb * ttl.math.broadcast(cb, dims=[0, 1]) + mb)
                with z_cb.wait() as zb:
                    with m_cb.reserve() as mx:
                        mx.store(ttl.math.reduce_max(zb, ob, dims=[1]))
                    with m_cb.wait() as mx, z_cb.reserve() as eb:
                        eb.store(ttl.math.exp(zb - ttl.math.broadcast(mx, dims=[1])))
                with z_cb.wait() as eb:
                    with d_cb.reserve() as db:
                        db.store(ttl.math.reduce_sum(eb, ob, dims=[1]))
                    with d_cb.wait() as db, p_cb.reserve() as pb:
                        pb.store(eb / ttl.math.broadcast(db, dims=[1]))

    @ttl.datamovement()
    def dm0():
        for r in my_rows():
            for cb_, src in ((s_cb, s[r:r + 1, 0:ct]), (mask_cb, mask[r:r + 1, 0:ct]), (scale_cb, scale[0:1, 0:1]),
                             (one_cb, one[0:1, 0:1])):
                with cb_.reserve() as blk:
                    tx = ttl.copy(src, blk)
                    tx.wait()

    @ttl.datamovement()
    def dm1():
        for r in my_rows():
            with p_cb.wait() as pb:
                tx = ttl.copy(pb, p[r:r + 1, 0:ct])
                tx.wait()


def attention_pipeline(q, kt, v, mask, scale, one, out):
    """out = softmax(scale * q @ kt + mask) @ v as three kernel calls; the score matrix and the probabilities are
    tensors of q's element type made here."""
    import torch

    s, dtype = q.shape[0], ttnn.to_torch(scale).dtype
    scores = ttnn.from_torch(torch.zeros((s, s), dtype=dtype))
    probs = ttnn.from_torch(torch.zeros((s, s), dtype=dtype))
    tile_matmul(q, kt, scores)
    masked_softmax_rows(scores, mask, scale, one, probs)
    tile_matmul(probs, v, out)

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

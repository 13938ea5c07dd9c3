"""tt-lang tile programs used by the parity tests: reductions.

`ttl.math.reduce_sum / reduce_max(expr, scaler, dims)` are specified
(docs/sphinx/specs/TTLangSpecification.md:750-755) but exist in neither the reference compiler
nor its simulator; on the simulator these programs run with the add-on in oracle/sim_addons.py.
Outputs are degenerate tensors ([1,N] row vector, [N,1] column, [1,1] scalar), the simulator's
idiom for a broadcast source (python/sim/copyhandlers.py:103-131).
"""
# type: ignore
import math

import ttl
import ttnn  # noqa: F401

N_CORES = 4


def _kernel(grid, fp32_dest_acc_en=False):
    if fp32_dest_acc_en:
        try:
            return ttl.kernel(grid=grid, fp32_dest_acc_en=True)
        except TypeError:
            pass
    return ttl.kernel(grid=grid)


def make_reduce(op, dims, fp32_dest_acc_en=False):
    """out = reduce_<op>(A, s, dims): each core reduces whole column strips (dims=[0]), whole row strips
    (dims=[1]) or, on one core, the whole tensor (dims=[0,1]) as ONE block."""
    red = getattr(ttl.math, "reduce_" + op)
    dims = list(dims)

    @_kernel((2, 2), fp32_dest_acc_en)
    def reduce_prog(a, s, out):
        rt, ct = a.shape[0] // 32, a.shape[1] // 32
        if dims == [0]:
            units, blk = ct, (rt, 1)
        elif dims == [1]:
            units, blk = rt, (1, ct)
        else:
            units, blk = 1, (rt, ct)
        per_core = math.ceil(units / N_CORES)
        a_cb = ttl.make_circular_buffer_like(a, shape=blk, buffer_factor=2)
        s_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

        def my_units():
            core = ttl.core(dims=1)
            return range(core * per_core, min((core + 1) * per_core, units))

        def a_slice(u):
            if dims == [0]:
                return a[0:rt, u:u + 1]
            if dims == [1]:
                return a[u:u + 1, 0:ct]
            return a[0:rt, 0:ct]

        def out_slice(u):
            if dims == [0]:
                return out[0:1, u:u + 1]
            if dims == [1]:
                return out[u:u + 1, 0:1]
            return out[0:1, 0:1]

        @ttl.compute()
        def compute():
            for _u in my_units():
                with a_cb.wait() as ab, s_cb.wait() as sb, o_cb.reserve() as ob:
                    ob.store(red(ab, sb, dims=dims))

        @ttl.datamovement()
        def dm0():
            for u in my_units():
                with a_cb.reserve() as ab:
                    tx = ttl.copy(a_slice(u), ab)
                    tx.wait()
                with s_cb.reserve() as sb:
                    tx = ttl.copy(s[0:1, 0:1], sb)
                    tx.wait()

        @ttl.datamovement()
        def dm1():
            for u in my_units():
                with o_cb.wait() as ob:
                    tx = ttl.copy(ob, out_slice(u))
                    tx.wait()

    return reduce_prog


def make_colsum_acc(rb, fp32_dest_acc_en=False):
    """out[0, :] = s * sum over rows of A, accumulated over blocks of `rb` row tiles with
    `store(..., acc=True)` into one reserved output block per column strip."""

    @_kernel((2, 2), fp32_dest_acc_en)
    def colsum_acc(a, s, out):
        rt, ct = a.shape[0] // 32, a.shape[1] // 32
        assert rt % rb == 0
        per_core = math.ceil(ct / N_CORES)
        a_cb = ttl.make_circular_buffer_like(a, shape=(rb, 1), buffer_factor=2)
        s_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

        def my_cols():
            core = ttl.core(dims=1)
            return range(core * per_core, min((core + 1) * per_core, ct))

        @ttl.compute()
        def compute():
            for _c in my_cols():
                with s_cb.wait() as sb, o_cb.reserve() as ob:
                    for _k in range(rt // rb):
                        with a_cb.wait() as ab:
                            ob.store(ttl.math.reduce_sum(ab, sb, dims=[0]), acc=True)

        @ttl.datamovement()
        def dm0():
            for c in my_cols():
                with s_cb.reserve() as sb:
                    tx = ttl.copy(s[0:1, 0:1], sb)
                    tx.wait()
                for k in range(rt // rb):
                    with a_cb.reserve() as ab:
                        tx = ttl.copy(a[k * rb:(k + 1) * rb, c:c + 1], ab)
                        tx.wait()

        @ttl.datamovement()
        def dm1():
            for c in my_cols():
                with o_cb.wait() as ob:
                    tx = ttl.copy(ob, out[0:1, c:c + 1])
                    tx.wait()

    return colsum_acc


def make_rowsum_exp(fp32_dest_acc_en=False):
    """out[:, 0] = s * sum_j exp(A[:, j]) * b[j]: an element-wise chain with a broadcast row vector,
    reduced over columns in the same kernel (the shape of a softmax denominator)."""

    @_kernel((2, 2), fp32_dest_acc_en)
    def rowsum_exp(a, b, s, out):
        rt, ct = a.shape[0] // 32, a.shape[1] // 32
        per_core = math.ceil(rt / N_CORES)
        a_cb = ttl.make_circular_buffer_like(a, shape=(1, ct), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, ct), buffer_factor=2)
        s_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

        def my_rows():
            core = ttl.core(dims=1)
            return range(core * per_core, min((core + 1) * per_core, rt))

        @ttl.compute()
        def compute():
            for _r in my_rows():
                with a_cb.wait() as ab, b_cb.wait() as bb, s_cb.wait() as sb, o_cb.reserve() as ob:
                    ob.store(ttl.math.reduce_sum(ttl.math.exp(ab) * ttl.math.broadcast(bb, dims=[0]), sb, dims=[1]))

        @ttl.datamovement()
        def dm0():
            for r in my_rows():
                with a_cb.reserve() as ab:
                    tx = ttl.copy(a[r:r + 1, 0:ct], ab)
                    tx.wait()
                with b_cb.reserve() as bb:
                    tx = ttl.copy(b[0:1, 0:ct], bb)
                    tx.wait()
                with s_cb.reserve() as sb:
                    tx = ttl.copy(s[0:1, 0:1], sb)
                    tx.wait()

        @ttl.datamovement()
        def dm1():
            for r in my_rows():
                with o_cb.wait() as ob:
                    tx = ttl.copy(ob, out[r:r + 1, 0:1])
                    tx.wait()

    return rowsum_exp


def make_softmax(fp32_dest_acc_en=False):
    """Row softmax as a tile program: y = exp(x - max_j x) / sum_j exp(x - max_j x), one row strip of
    tiles per step; the row maximum and the row sum travel through circular buffers of (1,1) blocks
    and are broadcast over the columns."""

    @_kernel((2, 2), fp32_dest_acc_en)
    def softmax(x, s, y):
        rt, ct = x.shape[0] // 32, x.shape[1] // 32
        per_core = math.ceil(rt / N_CORES)
        x_cb = ttl.make_circular_buffer_like(x, shape=(1, ct), buffer_factor=2)
        s_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
        m_cb = ttl.make_circular_buffer_like(x, shape=(1, 1), buffer_factor=2)
        e_cb = ttl.make_circular_buffer_like(x, shape=(1, ct), buffer_factor=2)
        d_cb = ttl.make_circular_buffer_like(x, shape=(1, 1), buffer_factor=2)
        y_cb = ttl.make_circular_buffer_like(y, shape=(1, ct), buffer_factor=2)

        def my_rows():
            core = ttl.core(dims=1)
            return range(core * per_core, min((core + 1) * per_core, rt))

        @ttl.compute()
        def compute():
            for _r in my_rows():
                with x_cb.wait() as xb, s_cb.wait() as sb:
                    with m_cb.reserve() as mb:
                        mb.store(ttl.math.reduce_max(xb, sb, dims=[1]))
                    with m_cb.wait() as mb, e_cb.reserve() as eb:
                        eb.store(ttl.math.exp(xb - ttl.math.broadcast(mb, dims=[1])))
                    with e_cb.wait() as eb:
                        with d_cb.reserve() as db:
                            db.store(ttl.math.reduce_sum(eb, sb, dims=[1]))
                        with d_cb.wait() as db, y_cb.reserve() as yb:
                            yb.store(eb / ttl.math.broadcast(db, dims=[1]))

        @ttl.datamovement()
        def dm0():
            for r in my_rows():
                with x_cb.reserve() as xb:
                    tx = ttl.copy(x[r:r + 1, 0:ct], xb)
                    tx.wait()
                with s_cb.reserve() as sb:
                    tx = ttl.copy(s[0:1, 0:1], sb)
                    tx.wait()

        @ttl.datamovement()
        def dm1():
            for r in my_rows():
                with y_cb.wait() as yb:
                    tx = ttl.copy(yb, y[r:r + 1, 0:ct])
                    tx.wait()

    return softmax


def make_standardize(fp32_dest_acc_en=False):
    """Row standardisation (the core of layer norm): c = x - mean_j x, y = c * rsqrt(mean_j c*c), with the
    scaler tile holding 1/N.  Two reductions, the second over an expression that reads the first."""

    @_kernel((2, 2), fp32_dest_acc_en)
    def standardize(x, s, y):
        rt, ct = x.shape[0] // 32, x.shape[1] // 32
        per_core = math.ceil(rt / N_CORES)
        x_cb = ttl.make_circular_buffer_like(x, shape=(1, ct), buffer_factor=2)
        s_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
        c_cb = ttl.make_circular_buffer_like(x, shape=(1, ct), buffer_factor=2)
        y_cb = ttl.make_circular_buffer_like(y, shape=(1, ct), buffer_factor=2)

        def my_rows():
            core = ttl.core(dims=1)
            return range(core * per_core, min((core + 1) * per_core, rt))

        @ttl.compute()
        def compute():
            for _r in my_rows():
                with x_cb.wait() as xb, s_cb.wait() as sb:
                    with c_cb.reserve() as cb:
                        cb.store(xb - ttl.math.broadcast(ttl.math.reduce_sum(xb, sb, dims=[1]), dims=[1]))
                    with c_cb.wait() as cb, y_cb.reserve() as yb:
                        var = ttl.math.reduce_sum(cb * cb, sb, dims=[1])
                        yb.store(cb * ttl.math.broadcast(ttl.math.rsqrt(var), dims=[1]))

        @ttl.datamovement()
        def dm0():
            for r in my_rows():
                with x_cb.reserve() as xb:
                    tx = ttl.copy(x[r:r + 1, 0:ct], xb)
                    tx.wait()
                with s_cb.reserve() as sb:
                    tx = ttl.copy(s[0:1, 0:1], sb)
                    tx.wait()

        @ttl.datamovement()
        def dm1():
            for r in my_rows():
                with y_cb.wait() as yb:
                    tx = ttl.copy(yb, y[r:r + 1, 0:ct])
                    tx.wait()

    return standardize

"""tt-lang tile programs used by the parity tests: element-wise and broadcast families.

Written against the DSL as the reference's examples use it (examples/eltwise_add.py:12-120,
examples/general_broadcast.py:24-156, examples/eltwise_pipe.py:12-162).  The same file runs
on the reference simulator (to produce golden vectors) and on the B200 backend.
"""
# type: ignore
import math

import ttl
import ttnn


@ttl.kernel(grid="auto")
def eltwise_add(a_in, b_in, out):
    """C = A + B, column-parallel over the 8x8 grid, (2,1)-tile blocks."""
    granularity = 2
    assert a_in.shape == b_in.shape == out.shape
    row_tiles = a_in.shape[0] // ttl.TILE_SHAPE[0]
    col_tiles = a_in.shape[1] // ttl.TILE_SHAPE[1]
    assert row_tiles % granularity == 0
    grid_h, grid_w = ttl.grid_size()
    cols_per_core = math.ceil(col_tiles / (grid_h * grid_w))
    a_cb = ttl.make_circular_buffer_like(a_in, shape=(granularity, 1), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b_in, shape=(granularity, 1), buffer_factor=2)
    out_cb = ttl.make_circular_buffer_like(out, shape=(granularity, 1), buffer_factor=2)

    @ttl.compute()
    def compute_func():
        core_num = ttl.core(dims=1)
        start = core_num * cols_per_core
        end = min(start + cols_per_core, col_tiles)
        for _ct in range(start, end):
            for _rt in range(row_tiles // granularity):
                a_block = a_cb.wait()
                b_block = b_cb.wait()
                out_block = out_cb.reserve()
                out_block.store(a_block + b_block)
                out_cb.push()
                a_cb.pop()
                b_cb.pop()

    @ttl.datamovement()
    def dm0():
        core_num = ttl.core(dims=1)
        start = core_num * cols_per_core
        end = min(start + cols_per_core, col_tiles)
        for ct in range(start, end):
            for rt in range(row_tiles // granularity):
                rs = slice(rt * granularity, (rt + 1) * granularity)
                cs = slice(ct, ct + 1)
                a_block = a_cb.reserve()
                tx = ttl.copy(a_in[rs, cs], a_block)
                tx.wait()
                a_cb.push()
                b_block = b_cb.reserve()
                tx = ttl.copy(b_in[rs, cs], b_block)
                tx.wait()
                b_cb.push()

    @ttl.datamovement()
    def dm1():
        core_num = ttl.core(dims=1)
        start = core_num * cols_per_core
        end = min(start + cols_per_core, col_tiles)
        for ct in range(start, end):
            for rt in range(row_tiles // granularity):
                rs = slice(rt * granularity, (rt + 1) * granularity)
                cs = slice(ct, ct + 1)
                out_block = out_cb.wait()
                tx = ttl.copy(out_block, out[rs, cs])
                tx.wait()
                out_cb.pop()


def _kernel(grid, fp32_dest_acc_en=False):
    """ttl.kernel with the compiler's fp32_dest_acc_en switch (python/ttl/ttl_api.py:1132) where
    the backend has it; the simulator's decorator only takes `grid` (python/sim/kernel.py:202)."""
    if fp32_dest_acc_en:
        try:
            return ttl.kernel(grid=grid, fp32_dest_acc_en=True)
        except TypeError:
            pass
    return ttl.kernel(grid=grid)


def _make_fused(fp32_dest_acc_en):
    @_kernel((8, 8), fp32_dest_acc_en)
    def fused_exp_bcast(a, s, b, c, y):
        """Y = relu(exp(s * A) * b + C): s is a [1,1] scalar tile, b a [1,N] row vector
        broadcast over rows; blocks of up to 4x4 tiles."""
        grid_x, grid_y = ttl.grid_size(dims=2)
        row_tiles = a.shape[0] // 32
        col_tiles = a.shape[1] // 32
        rb = 4 if row_tiles % (4 * grid_x) == 0 else 1
        cb = 4 if col_tiles % (4 * grid_y) == 0 else 1
        rows_per_core = math.ceil(row_tiles / rb / grid_x)
        cols_per_core = math.ceil(col_tiles / cb / grid_y)
        a_cb = ttl.make_circular_buffer_like(a, shape=(rb, cb), buffer_factor=2)
        s_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, cb), buffer_factor=2)
        c_cb = ttl.make_circular_buffer_like(c, shape=(rb, cb), buffer_factor=2)
        y_cb = ttl.make_circular_buffer_like(y, shape=(rb, cb), buffer_factor=2)

        def my_blocks():
            core_x, core_y = ttl.core(dims=2)
            for i in range(rows_per_core):
                r = core_x * rows_per_core + i
                if (r + 1) * rb > row_tiles:
                    continue
                for j in range(cols_per_core):
                    col = core_y * cols_per_core + j
                    if (col + 1) * cb > col_tiles:
                        continue
                    yield r * rb, (r + 1) * rb, col * cb, (col + 1) * cb

        @ttl.compute()
        def fused_compute():
            for _ in my_blocks():
                with (a_cb.wait() as a_blk, s_cb.wait() as s_blk, b_cb.wait() as b_blk,
                      c_cb.wait() as c_blk, y_cb.reserve() as y_blk):
                    scaled = a_blk * ttl.math.broadcast(s_blk, dims=[0, 1])
                    e = ttl.math.exp(scaled)
                    y_blk.store(ttl.math.relu(e * ttl.math.broadcast(b_blk, dims=[0]) + c_blk))

        @ttl.datamovement()
        def fused_read():
            for r0, r1, c0, c1 in my_blocks():
                with (a_cb.reserve() as a_blk, s_cb.reserve() as s_blk, b_cb.reserve() as b_blk,
                      c_cb.reserve() as c_blk):
                    txs = [ttl.copy(a[r0:r1, c0:c1], a_blk), ttl.copy(s[0:1, 0:1], s_blk),
                           ttl.copy(b[0:1, c0:c1], b_blk), ttl.copy(c[r0:r1, c0:c1], c_blk)]
                    for tx in txs:
                        tx.wait()

        @ttl.datamovement()
        def fused_write():
            for r0, r1, c0, c1 in my_blocks():
                with y_cb.wait() as y_blk:
                    tx = ttl.copy(y_blk, y[r0:r1, c0:c1])
                    tx.wait()

    return fused_exp_bcast


fused_exp_bcast = _make_fused(False)        # every op rounds to the tensor dtype (simulator-native)
fused_exp_bcast_f32acc = _make_fused(True)  # fp32 intermediates, one final rounding


@ttl.kernel(grid=(2, 2))
def mul_add_bcast(a, b, c, y):
    """Y = A * B + C where B and C may be full, a row vector [1,N] / one tile row [32,N],
    a column [M,1] / one tile column [M,32], or a scalar [1,1] (general_broadcast.py style)."""
    R = C = 2
    grid_x, grid_y = ttl.grid_size(dims=2)
    rows_per_core = a.shape[0] // 32 // grid_x // R
    cols_per_core = a.shape[1] // 32 // grid_y // C

    def tiles(t):
        return (R if t.shape[0] > 32 else 1, C if t.shape[1] > 32 else 1)

    bt, ct = tiles(b), tiles(c)
    a_cb = ttl.make_circular_buffer_like(a, shape=(R, C), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b, shape=bt, buffer_factor=2)
    c_cb = ttl.make_circular_buffer_like(c, shape=ct, buffer_factor=2)
    y_cb = ttl.make_circular_buffer_like(y, shape=(R, C), buffer_factor=2)

    def bc(blk, t):
        dims = [d for d in (0, 1) if t[d] == 1 and (R, C)[d] > 1]
        return ttl.math.broadcast(blk, dims=dims) if dims else blk

    @ttl.compute()
    def compute():
        for _ in range(rows_per_core * cols_per_core):
            with a_cb.wait() as a_blk, b_cb.wait() as b_blk, c_cb.wait() as c_blk, y_cb.reserve() as y_blk:
                y_blk.store(a_blk * bc(b_blk, bt) + bc(c_blk, ct))

    def region(t, tl, r0, c0):
        rr = (r0, r0 + R) if tl[0] == R and t.shape[0] > 32 else (0, 1)
        cc = (c0, c0 + C) if tl[1] == C and t.shape[1] > 32 else (0, 1)
        return slice(*rr), slice(*cc)

    @ttl.datamovement()
    def read():
        core_x, core_y = ttl.core(dims=2)
        for i in range(rows_per_core):
            for j in range(cols_per_core):
                r0 = (core_x * rows_per_core + i) * R
                c0 = (core_y * cols_per_core + j) * C
                with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk, c_cb.reserve() as c_blk:
                    t1 = ttl.copy(a[r0:r0 + R, c0:c0 + C], a_blk)
                    t2 = ttl.copy(b[region(b, bt, r0, c0)], b_blk)
                    t3 = ttl.copy(c[region(c, ct, r0, c0)], c_blk)
                    t1.wait()
                    t2.wait()
                    t3.wait()

    @ttl.datamovement()
    def write():
        core_x, core_y = ttl.core(dims=2)
        for i in range(rows_per_core):
            for j in range(cols_per_core):
                r0 = (core_x * rows_per_core + i) * R
                c0 = (core_y * cols_per_core + j) * C
                with y_cb.wait() as y_blk:
                    tx = ttl.copy(y_blk, y[r0:r0 + R, c0:c0 + C])
                    tx.wait()


def make_unary_chain(op_names, fp32_dest_acc_en=False):
    """Y = opN(...op1(A)...) + B on 1x1-tile blocks, single core; op names from ttl.math, or
    (name, scalar parameters...) for functions such as leaky_relu(x, slope)."""
    @_kernel((1, 1), fp32_dest_acc_en)
    def unary_chain(a, b, y):
        rt, ct = a.shape[0] // 32, a.shape[1] // 32
        a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
        y_cb = ttl.make_circular_buffer_like(y, shape=(1, 1), buffer_factor=2)

        @ttl.compute()
        def compute():
            for _ in range(rt * ct):
                with a_cb.wait() as a_blk, b_cb.wait() as b_blk, y_cb.reserve() as y_blk:
                    v = a_blk
                    for name in op_names:
                        if isinstance(name, (tuple, list)):
                            v = getattr(ttl.math, name[0])(v, *name[1:])
                        else:
                            v = getattr(ttl.math, name)(v)
                    y_blk.store(v + b_blk)

        @ttl.datamovement()
        def read():
            for r in range(rt):
                for c in range(ct):
                    with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                        t1 = ttl.copy(a[r, c], a_blk)
                        t2 = ttl.copy(b[r, c], b_blk)
                        t1.wait()
                        t2.wait()

        @ttl.datamovement()
        def write():
            for r in range(rt):
                for c in range(ct):
                    with y_cb.wait() as y_blk:
                        tx = ttl.copy(y_blk, y[r, c])
                        tx.wait()

    return unary_chain


@ttl.kernel(grid=(1, 1))
def sum_of_products(a, b, c, d, y):
    """Y = (A*B - C*D) / (A*A + D): needs temporaries (exercises the expression stack)."""
    rt, ct = a.shape[0] // 32, a.shape[1] // 32
    cbs = [ttl.make_circular_buffer_like(t, shape=(1, ct), buffer_factor=2) for t in (a, b, c, d)]
    a_cb, b_cb, c_cb, d_cb = cbs
    y_cb = ttl.make_circular_buffer_like(y, shape=(1, ct), buffer_factor=2)

    @ttl.compute()
    def compute():
        for _ in range(rt):
            with a_cb.wait() as a_blk, b_cb.wait() as b_blk, c_cb.wait() as c_blk, d_cb.wait() as d_blk:
                with y_cb.reserve() as y_blk:
                    y_blk.store((a_blk * b_blk - c_blk * d_blk) / (a_blk * a_blk + d_blk))

    @ttl.datamovement()
    def read():
        for r in range(rt):
            with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk, c_cb.reserve() as c_blk, d_cb.reserve() as d_blk:
                txs = [ttl.copy(t[r:r + 1, 0:ct], blk) for t, blk in ((a, a_blk), (b, b_blk), (c, c_blk), (d, d_blk))]
                for tx in txs:
                    tx.wait()

    @ttl.datamovement()
    def write():
        for r in range(rt):
            with y_cb.wait() as y_blk:
                tx = ttl.copy(y_blk, y[r:r + 1, 0:ct])
                tx.wait()


@ttl.kernel(grid="auto")
def eltwise_pipe(a_in, b_in, c_tile, out):
    """out = A * B + bcast(C tile) on the cores of one multicast pipe: core (0,0) reads the
    C tile and multicasts it to cores (0,1..3); only those four cores compute
    (examples/eltwise_pipe.py:55-162)."""
    granularity = 2
    row_tiles = a_in.shape[0] // ttl.TILE_SHAPE[0]
    col_tiles = a_in.shape[1] // ttl.TILE_SHAPE[1]
    grid_h, grid_w = ttl.grid_size()
    cols_per_core = math.ceil(col_tiles / (grid_h * grid_w))
    a_cb = ttl.make_circular_buffer_like(a_in, shape=(granularity, 1), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b_in, shape=(granularity, 1), buffer_factor=2)
    c_cb = ttl.make_circular_buffer_like(c_tile, shape=(1, 1), buffer_factor=2)
    out_cb = ttl.make_circular_buffer_like(out, shape=(granularity, 1), buffer_factor=2)
    pipe = ttl.Pipe((0, 0), (0, slice(1, 4)))
    pipe_net = ttl.PipeNet([pipe])

    @ttl.compute()
    def compute_func():
        if not pipe.has_current_core():
            return
        core_num = ttl.core(dims=1)
        start = core_num * cols_per_core
        end = min(start + cols_per_core, col_tiles)
        c_block = c_cb.wait()
        for _ct in range(start, end):
            for _rt in range(row_tiles // granularity):
                a_block = a_cb.wait()
                b_block = b_cb.wait()
                out_block = out_cb.reserve()
                out_block.store(a_block * b_block + ttl.math.broadcast(c_block, dims=[0]))
                out_cb.push()
                a_cb.pop()
                b_cb.pop()
        c_cb.pop()

    @ttl.datamovement()
    def dm0():
        if not pipe.has_current_core():
            return
        core_num = ttl.core(dims=1)
        with c_cb.reserve() as c_block:
            def pipe_src(pipe_id):
                tx = ttl.copy(c_tile[slice(0, 1), slice(0, 1)], c_block)
                tx.wait()
                tx = ttl.copy(c_block, pipe_id)
                tx.wait()

            def pipe_dst(pipe_id):
                tx = ttl.copy(pipe_id, c_block)
                tx.wait()

            pipe_net.if_src(pipe_src)
            pipe_net.if_dst(pipe_dst)
        start = core_num * cols_per_core
        end = min(start + cols_per_core, col_tiles)
        for ct in range(start, end):
            for rt in range(row_tiles // granularity):
                rs = slice(rt * granularity, (rt + 1) * granularity)
                cs = slice(ct, ct + 1)
                a_block = a_cb.reserve()
                tx = ttl.copy(a_in[rs, cs], a_block)
                tx.wait()
                a_cb.push()
                b_block = b_cb.reserve()
                tx = ttl.copy(b_in[rs, cs], b_block)
                tx.wait()
                b_cb.push()

    @ttl.datamovement()
    def dm1():
        if not pipe.has_current_core():
            return
        core_num = ttl.core(dims=1)
        start = core_num * cols_per_core
        end = min(start + cols_per_core, col_tiles)
        for ct in range(start, end):
            for rt in range(row_tiles // granularity):
                rs = slice(rt * granularity, (rt + 1) * granularity)
                cs = slice(ct, ct + 1)
                out_block = out_cb.wait()
                tx = ttl.copy(out_block, out[rs, cs])
                tx.wait()
                out_cb.pop()


@ttl.kernel(grid=(2, 1))
def intermediate_cb(a, b, y):
    """Y = exp(A) * B with the exponential staged through an intermediate circular buffer that the
    compute thread both fills and drains (the pattern of test/python/test_intermediate_cb.py)."""
    rt, ct = a.shape[0] // 32, a.shape[1] // 32
    n_cores = ttl.grid_size(dims=1)
    a_cb = ttl.make_circular_buffer_like(a, shape=(1, ct), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b, shape=(1, ct), buffer_factor=2)
    t_cb = ttl.make_circular_buffer_like(a, shape=(1, ct), buffer_factor=2)
    y_cb = ttl.make_circular_buffer_like(y, shape=(1, ct), buffer_factor=2)

    def my_rows():
        return range(ttl.core(dims=1), rt, n_cores)

    @ttl.compute()
    def compute():
        for _ in my_rows():
            with a_cb.wait() as a_blk, t_cb.reserve() as t_blk:
                t_blk.store(ttl.math.exp(a_blk))
            with t_cb.wait() as t_blk, b_cb.wait() as b_blk, y_cb.reserve() as y_blk:
                y_blk.store(t_blk * b_blk)

    @ttl.datamovement()
    def read():
        for r in my_rows():
            with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                t1 = ttl.copy(a[r:r + 1, 0:ct], a_blk)
                t2 = ttl.copy(b[r:r + 1, 0:ct], b_blk)
                t1.wait()
                t2.wait()

    @ttl.datamovement()
    def write():
        for r in my_rows():
            with y_cb.wait() as y_blk:
                tx = ttl.copy(y_blk, y[r:r + 1, 0:ct])
                tx.wait()


def make_hw_broadcast(dims, in_block, out_block):
    """Compiler-style broadcast of FULL tiles (test/python/test_bcast_ops.py:60-84): the first row
    (dims=[0]) / first column (dims=[1]) / element [0,0] (dims=[0,1]) of every source tile is spread
    over the tile; a source block of one tile along a dim expands to the output block.  Computes
    out = x * 2 + broadcast(b) on one block.  Only meaningful with the hardware broadcast switch on."""

    @ttl.kernel(grid=(1, 1))
    def hw_broadcast(x, b, out):
        x_cb = ttl.make_circular_buffer_like(x, shape=out_block, buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=in_block, buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(out, shape=out_block, buffer_factor=2)

        @ttl.compute()
        def compute():
            with x_cb.wait() as xb, b_cb.wait() as bb, o_cb.reserve() as ob:
                ob.store(xb + xb + ttl.math.broadcast(bb, ob, dims=dims))

        @ttl.datamovement()
        def reader():
            with x_cb.reserve() as xb, b_cb.reserve() as bb:
                tx = ttl.copy(x[0:out_block[0], 0:out_block[1]], xb)
                tb = ttl.copy(b[0:in_block[0], 0:in_block[1]], bb)
                tx.wait()
                tb.wait()

        @ttl.datamovement()
        def writer():
            with o_cb.wait() as ob:
                tx = ttl.copy(ob, out[0:out_block[0], 0:out_block[1]])
                tx.wait()

    return hw_broadcast


def make_operator(name, exponent=None, fp32_dest_acc_en=False):
    """Y = A <op> B for the Python operators `//`, `%`, `**` on blocks, or Y = A ** exponent with an integer
    exponent (python/sim/block.py:975-1010); (1, ct)-tile blocks, rows dealt out over a 2x2 grid."""
    import operator
    fn = {"floordiv": operator.floordiv, "mod": operator.mod, "pow": operator.pow}[name]

    @_kernel((2, 2), fp32_dest_acc_en)
    def operator_prog(a, b, y):
        rt, ct = a.shape[0] // 32, a.shape[1] // 32
        n_cores = 4
        a_cb = ttl.make_circular_buffer_like(a, shape=(1, ct), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, ct), buffer_factor=2)
        y_cb = ttl.make_circular_buffer_like(y, shape=(1, ct), buffer_factor=2)

        def my_rows():
            return range(ttl.core(dims=1), rt, n_cores)

        @ttl.compute()
        def compute():
            for _r in my_rows():
                with a_cb.wait() as a_blk, b_cb.wait() as b_blk, y_cb.reserve() as y_blk:
                    if exponent is None:
                        y_blk.store(fn(a_blk, b_blk))
                    else:
                        y_blk.store(a_blk ** exponent + b_blk)

        @ttl.datamovement()
        def read():
            for r in my_rows():
                with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                    t1 = ttl.copy(a[r:r + 1, 0:ct], a_blk)
                    t2 = ttl.copy(b[r:r + 1, 0:ct], b_blk)
                    t1.wait()
                    t2.wait()

        @ttl.datamovement()
        def write():
            for r in my_rows():
                with y_cb.wait() as y_blk:
                    tx = ttl.copy(y_blk, y[r:r + 1, 0:ct])
                    tx.wait()

    return operator_prog

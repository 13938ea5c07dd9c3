"""tt-lang matmul tile programs used by the parity tests (examples/singlecore_matmul.py:11-69,
examples/multicore_matmul.py:28-139): `out_blk.store(a_blk @ b_blk, acc=True)` over the K tiles."""
# type: ignore
import ttl
import ttnn


@ttl.kernel(grid=(1, 1))
def singlecore_matmul(a, b, out):
    assert a.shape[1] == b.shape[0], "Incompatible matrix shapes for multiplication."
    assert a.shape[0] == out.shape[0], "Output matrix has incorrect number of rows."
    Mt, Kt, Nt = a.shape[0] // ttnn.TILE_SIZE, a.shape[1] // ttnn.TILE_SIZE, b.shape[1] // ttnn.TILE_SIZE
    a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
    out_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

    @ttl.compute()
    def mm_compute():
        for _ in range(Mt):
            for _ in range(Nt):
                with out_cb.reserve() as out_blk:
                    for _ in range(Kt):
                        with a_cb.wait() as a_blk, b_cb.wait() as b_blk:
                            out_blk.store(a_blk @ b_blk, acc=True)

    @ttl.datamovement()
    def mm_reader():
        for m in range(Mt):
            for n in range(Nt):
                for k in range(Kt):
                    with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                        a_wr = ttl.copy(a[m, k], a_blk)
                        b_wr = ttl.copy(b[k, n], b_blk)
                        a_wr.wait()
                        b_wr.wait()

    @ttl.datamovement()
    def mm_writer():
        for m in range(Mt):
            for n in range(Nt):
                with out_cb.wait() as out_blk:
                    tx = ttl.copy(out_blk, out[m, n])
                    tx.wait()


def _cores(core_range_set):
    return sum((r.end.x - r.start.x + 1) * (r.end.y - r.start.y + 1) for r in core_range_set.ranges())


@ttl.kernel(grid=(13, 10))
def multicore_matmul(a, b, out):
    """Output tiles split over a 13x10 grid with ttnn.split_work_to_cores."""
    Kt, Nt = a.shape[1] // ttnn.TILE_SIZE, b.shape[1] // ttnn.TILE_SIZE
    total = (a.shape[0] * b.shape[1]) // (ttnn.TILE_SIZE * ttnn.TILE_SIZE)
    a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
    out_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)
    y_size, x_size = ttl.grid_size(dims=2)
    (_, _all, g1, g2, w1, w2) = ttnn.split_work_to_cores(ttnn.CoreCoord(x_size, y_size), total, row_wise=True)
    n1, n2 = _cores(g1), _cores(g2)

    def tiles_of(core_id):
        if core_id < n1:
            return core_id * w1, w1
        if core_id < n1 + n2:
            return n1 * w1 + (core_id - n1) * w2, w2
        return 0, 0

    @ttl.compute()
    def mm_compute():
        _, num = tiles_of(ttl.core(dims=1))
        for _ in range(num):
            with out_cb.reserve() as out_blk:
                for _ in range(Kt):
                    with a_cb.wait() as a_blk, b_cb.wait() as b_blk:
                        out_blk.store(a_blk @ b_blk, acc=True)

    @ttl.datamovement()
    def mm_reader():
        start, num = tiles_of(ttl.core(dims=1))
        for t in range(start, start + num):
            for k in range(Kt):
                with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                    a_wr = ttl.copy(a[t // Nt, k], a_blk)
                    b_wr = ttl.copy(b[k, t % Nt], b_blk)
                    a_wr.wait()
                    b_wr.wait()

    @ttl.datamovement()
    def mm_writer():
        start, num = tiles_of(ttl.core(dims=1))
        for t in range(start, start + num):
            with out_cb.wait() as out_blk:
                tx = ttl.copy(out_blk, out[t // Nt, t % Nt])
                tx.wait()


def make_blocked_matmul(bm, bn, grid=(4, 4)):
    """Output blocks of (bm, bn) tiles: each K step is the outer product of a (bm,1) column of A
    tiles and a (1,bn) row of B tiles, the multi-tile form the simulator evaluates as a block
    matmul (python/sim/block.py:870-920)."""

    @ttl.kernel(grid=grid)
    def blocked_matmul(a, b, out):
        Mt, Kt, Nt = a.shape[0] // 32, a.shape[1] // 32, b.shape[1] // 32
        assert Mt % bm == 0 and Nt % bn == 0
        blocks = [(i, j) for i in range(Mt // bm) for j in range(Nt // bn)]
        n_cores = ttl.grid_size(dims=1)
        a_cb = ttl.make_circular_buffer_like(a, shape=(bm, 1), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, bn), buffer_factor=2)
        out_cb = ttl.make_circular_buffer_like(out, shape=(bm, bn), buffer_factor=2)

        def mine():
            return blocks[ttl.core(dims=1)::n_cores]

        @ttl.compute()
        def mm_compute():
            for _ in mine():
                with out_cb.reserve() as out_blk:
                    for _ in range(Kt):
                        with a_cb.wait() as a_blk, b_cb.wait() as b_blk:
                            out_blk.store(a_blk @ b_blk, acc=True)

        @ttl.datamovement()
        def mm_reader():
            for i, j in mine():
                for k in range(Kt):
                    with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                        a_wr = ttl.copy(a[i * bm:(i + 1) * bm, k:k + 1], a_blk)
                        b_wr = ttl.copy(b[k:k + 1, j * bn:(j + 1) * bn], b_blk)
                        a_wr.wait()
                        b_wr.wait()

        @ttl.datamovement()
        def mm_writer():
            for i, j in mine():
                with out_cb.wait() as out_blk:
                    tx = ttl.copy(out_blk, out[i * bm:(i + 1) * bm, j * bn:(j + 1) * bn])
                    tx.wait()

    return blocked_matmul


@ttl.kernel(grid=(1, 1))
def matmul_bias(a, b, c, out):
    """Y = A @ B + C as in the specification's matmul example (2-D operands):
    `y_blk.store(c_blk, acc=True)` and then `y_blk.store(a_blk @ b_blk, acc=True)` over the K tiles."""
    Mt, Kt, Nt = a.shape[0] // ttnn.TILE_SIZE, a.shape[1] // ttnn.TILE_SIZE, b.shape[1] // ttnn.TILE_SIZE
    a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
    c_cb = ttl.make_circular_buffer_like(c, shape=(1, 1), buffer_factor=2)
    y_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

    @ttl.compute()
    def mm_compute():
        for _ in range(Mt):
            for _ in range(Nt):
                with y_cb.reserve() as y_blk:
                    with c_cb.wait() as c_blk:
                        y_blk.store(c_blk, acc=True)
                    for _ in range(Kt):
                        with a_cb.wait() as a_blk, b_cb.wait() as b_blk:
                            y_blk.store(a_blk @ b_blk, acc=True)

    @ttl.datamovement()
    def mm_reader():
        for m in range(Mt):
            for n in range(Nt):
                with c_cb.reserve() as c_blk:
                    c_xf = ttl.copy(c[m, n], c_blk)
                    c_xf.wait()
                for k in range(Kt):
                    with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                        a_xf = ttl.copy(a[m, k], a_blk)
                        b_xf = ttl.copy(b[k, n], b_blk)
                        a_xf.wait()
                        b_xf.wait()

    @ttl.datamovement()
    def mm_writer():
        for m in range(Mt):
            for n in range(Nt):
                with y_cb.wait() as y_blk:
                    y_xf = ttl.copy(y_blk, out[m, n])
                    y_xf.wait()


def _kernel(grid, fp32_dest_acc_en=False):
    if fp32_dest_acc_en:
        try:
            return ttl.kernel(grid=grid, fp32_dest_acc_en=True)
        except TypeError:
            pass
    return ttl.kernel(grid=grid)


def make_linear(act, fp32_dest_acc_en=False):
    """Y = act(A @ B + bias) like `linear_relu`, for any unary function of ttl.math; with fp32_dest_acc_en the
    bias and the activation are applied to the fp32 product (on the B200 backend: inside the GEMM)."""
    fn = getattr(ttl.math, act)

    @_kernel((1, 1), fp32_dest_acc_en)
    def linear(a, b, bias, out):
        Mt, Kt, Nt = a.shape[0] // ttnn.TILE_SIZE, a.shape[1] // ttnn.TILE_SIZE, b.shape[1] // ttnn.TILE_SIZE
        a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
        v_cb = ttl.make_circular_buffer_like(bias, shape=(1, 1), buffer_factor=2)
        p_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)
        y_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

        @ttl.compute()
        def mm_compute():
            for _ in range(Mt):
                for _ in range(Nt):
                    with p_cb.reserve() as p_blk:
                        for _ in range(Kt):
                            with a_cb.wait() as a_blk, b_cb.wait() as b_blk:
                                p_blk.store(a_blk @ b_blk, acc=True)
                    with p_cb.wait() as p_blk, v_cb.wait() as v_blk, y_cb.reserve() as y_blk:
                        y_blk.store(fn(p_blk + ttl.math.broadcast(v_blk, dims=[0])))

        @ttl.datamovement()
        def mm_reader():
            for m in range(Mt):
                for n in range(Nt):
                    for k in range(Kt):
                        with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                            a_xf = ttl.copy(a[m, k], a_blk)
                            b_xf = ttl.copy(b[k, n], b_blk)
                            a_xf.wait()
                            b_xf.wait()
                    with v_cb.reserve() as v_blk:
                        v_xf = ttl.copy(bias[0, n], v_blk)
                        v_xf.wait()

        @ttl.datamovement()
        def mm_writer():
            for m in range(Mt):
                for n in range(Nt):
                    with y_cb.wait() as y_blk:
                        y_xf = ttl.copy(y_blk, out[m, n])
                        y_xf.wait()

    return linear


@ttl.kernel(grid=(1, 1))
def linear_relu(a, b, bias, out):
    """Y = relu(A @ B + bias), bias a [1, N] row vector: the product is accumulated over the K tiles into a
    block of an intermediate circular buffer, then bias and activation are applied on the way to the output."""
    Mt, Kt, Nt = a.shape[0] // ttnn.TILE_SIZE, a.shape[1] // ttnn.TILE_SIZE, b.shape[1] // ttnn.TILE_SIZE
    a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1), buffer_factor=2)
    b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
    v_cb = ttl.make_circular_buffer_like(bias, shape=(1, 1), buffer_factor=2)
    p_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)
    y_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

    @ttl.compute()
    def mm_compute():
        for _ in range(Mt):
            for _ in range(Nt):
                with p_cb.reserve() as p_blk:
                    for _ in range(Kt):
                        with a_cb.wait() as a_blk, b_cb.wait() as b_blk:
                            p_blk.store(a_blk @ b_blk, acc=True)
                with p_cb.wait() as p_blk, v_cb.wait() as v_blk, y_cb.reserve() as y_blk:
                    y_blk.store(ttl.math.relu(p_blk + ttl.math.broadcast(v_blk, dims=[0])))

    @ttl.datamovement()
    def mm_reader():
        for m in range(Mt):
            for n in range(Nt):
                for k in range(Kt):
                    with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                        a_xf = ttl.copy(a[m, k], a_blk)
                        b_xf = ttl.copy(b[k, n], b_blk)
                        a_xf.wait()
                        b_xf.wait()
                with v_cb.reserve() as v_blk:
                    v_xf = ttl.copy(bias[0, n], v_blk)
                    v_xf.wait()

    @ttl.datamovement()
    def mm_writer():
        for m in range(Mt):
            for n in range(Nt):
                with y_cb.wait() as y_blk:
                    y_xf = ttl.copy(y_blk, out[m, n])
                    y_xf.wait()


def make_kblock_matmul(bm, bk, bn, grid=(2, 2)):
    """Blocks of (bm, bk) @ (bk, bn) tiles accumulated over K in steps of bk tiles: the specification's block
    dot product (docs/sphinx/specs/TTLangSpecification.md:694) as the reference's reuse matmul uses it
    (examples/metal_examples/multicore_reuse_matmul/ttlang/multicore_reuse_matmul.py:59-70)."""

    @ttl.kernel(grid=grid)
    def kblock_matmul(a, b, out):
        Mt, Kt, Nt = a.shape[0] // 32, a.shape[1] // 32, b.shape[1] // 32
        assert Mt % bm == 0 and Nt % bn == 0 and Kt % bk == 0
        blocks = [(i, j) for i in range(Mt // bm) for j in range(Nt // bn)]
        n_cores = ttl.grid_size(dims=1)
        a_cb = ttl.make_circular_buffer_like(a, shape=(bm, bk), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(bk, bn), buffer_factor=2)
        out_cb = ttl.make_circular_buffer_like(out, shape=(bm, bn), buffer_factor=1)

        def mine():
            return blocks[ttl.core(dims=1)::n_cores]

        @ttl.compute()
        def mm_compute():
            for _ in mine():
                with out_cb.reserve() as out_blk:
                    for _ in range(Kt // bk):
                        with a_cb.wait() as a_blk, b_cb.wait() as b_blk:
                            out_blk.store(a_blk @ b_blk, acc=True)

        @ttl.datamovement()
        def mm_reader():
            for i, j in mine():
                for k in range(0, Kt, bk):
                    with a_cb.reserve() as a_blk, b_cb.reserve() as b_blk:
                        a_wr = ttl.copy(a[i * bm:(i + 1) * bm, k:k + bk], a_blk)
                        b_wr = ttl.copy(b[k:k + bk, j * bn:(j + 1) * bn], b_blk)
                        a_wr.wait()
                        b_wr.wait()

        @ttl.datamovement()
        def mm_writer():
            for i, j in mine():
                with out_cb.wait() as out_blk:
                    tx = ttl.copy(out_blk, out[i * bm:(i + 1) * bm, j * bn:(j + 1) * bn])
                    tx.wait()

    return kblock_matmul

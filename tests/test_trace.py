"""Host-side logic: tracing tile programs and recognising them (no GPU needed).

Mirrors what the reference pins in test/sim (test_cb.py, test_copy.py, test_program.py,
test_math.py): circular-buffer contract errors, copy shape validation, broadcast validation,
deadlock reporting, per-core isolation - here on the symbolic tracer.
"""

import pytest
import torch

import cases


@pytest.fixture()
def tt(backend):
    import ttl
    import ttnn
    return ttl, ttnn


def _t(ttnn, shape, dtype=torch.bfloat16):
    return ttnn.from_torch(torch.zeros(shape, dtype=dtype))


def test_config1_add_plan(backend, tt):
    _, mods = backend
    ttl, ttnn = tt
    a, b, o = (_t(ttnn, (1024, 1024)) for _ in range(3))
    plan = mods["eltwise"].eltwise_add.plan(a, b, o)
    d = plan.describe()
    assert len(d) == 1 and d[0]["rect_tiles"] == (0, 32, 0, 32)
    assert d[0]["ops"] == [("load", 0), ("add", 1)] and d[0]["round_each_op"] is True
    # second call hits the per-signature cache
    assert mods["eltwise"].eltwise_add.plan(a, b, o) is plan


def test_fused_plan_modes_and_operand_addressing(backend, tt):
    from ttl_b200 import capi
    _, mods = backend
    ttl, ttnn = tt
    a, c, y = (_t(ttnn, (256, 512)) for _ in range(3))
    s, b = _t(ttnn, (1, 1)), _t(ttnn, (1, 512))
    d = mods["eltwise"].fused_exp_bcast_f32acc.plan(a, s, b, c, y).describe()[0]
    assert d["round_each_op"] is False
    assert [op for op, _ in d["ops"]] == ["load", "mul", "exp", "mul", "add", "relu"]
    modes = {i[0]: (i[1], i[3]) for i in d["inputs"]}
    assert modes[0] == (capi.IDX_SAME, capi.IDX_SAME)
    assert modes[1] == (capi.IDX_ZERO, capi.IDX_ZERO)   # scalar tile
    assert modes[2] == (capi.IDX_ZERO, capi.IDX_SAME)   # row vector
    assert mods["eltwise"].fused_exp_bcast.plan(a, s, b, c, y).describe()[0]["round_each_op"] is True


def test_pipe_program_covers_only_pipe_cores(backend, tt):
    _, mods = backend
    ttl, ttnn = tt
    a, b, o = (_t(ttnn, (128, 2048)) for _ in range(3))
    d = mods["eltwise"].eltwise_pipe.plan(a, b, _t(ttnn, (32, 32)), o).describe()
    assert len(d) == 1 and d[0]["rect_tiles"] == (0, 4, 0, 4)


@pytest.mark.parametrize("name", ["singlecore_matmul", "multicore_matmul"])
def test_matmul_recognised(backend, tt, name):
    _, mods = backend
    ttl, ttnn = tt
    a, b, o = _t(ttnn, (256, 192)), _t(ttnn, (192, 128)), _t(ttnn, (256, 128))
    d = getattr(mods["matmul"], name).plan(a, b, o).describe()
    assert d == [{"kind": "matmul_bf16", "a": 0, "b": 1, "out": 2, "rect_tiles": (0, 8, 0, 4), "k_tiles": 6}]


def test_matmul_with_bias_recognised(backend, tt):
    """The specification's matmul with bias (a store of the C block before the K loop) becomes one GEMM
    launch with the bias operand; a bias block that is not the output tile's block is refused."""
    _, mods = backend
    ttl, ttnn = tt
    a, b = _t(ttnn, (64, 96)), _t(ttnn, (96, 128))
    c, o = _t(ttnn, (64, 128)), _t(ttnn, (64, 128))
    d = mods["matmul"].matmul_bias.plan(a, b, c, o).describe()
    assert d == [{"kind": "matmul_bf16", "a": 0, "b": 1, "out": 3, "rect_tiles": (0, 2, 0, 4), "k_tiles": 3, "bias": 2}]


def test_blocked_matmul_recognised_and_tilewise_product_rejected(backend, tt):
    from ttl_b200 import Unsupported
    _, mods = backend
    ttl, ttnn = tt
    a, b, o = _t(ttnn, (256, 256)), _t(ttnn, (256, 256)), _t(ttnn, (256, 256))
    d = mods["matmul"].make_blocked_matmul(2, 4).plan(a, b, o).describe()
    assert d[0]["kind"] == "matmul_bf16" and d[0]["rect_tiles"] == (0, 8, 0, 8)

    @ttl.kernel(grid=(1, 1))
    def tilewise(a, b, out):   # (2,2)@(2,2): a tile-wise product in the simulator, not a block matmul
        cbs = [ttl.make_circular_buffer_like(t, shape=(2, 2)) for t in (a, b, out)]

        @ttl.compute()
        def c():
            with cbs[0].wait() as x, cbs[1].wait() as y, cbs[2].reserve() as z:
                z.store(x @ y)

        @ttl.datamovement()
        def r():
            with cbs[0].reserve() as x, cbs[1].reserve() as y:
                t1 = ttl.copy(a[0:2, 0:2], x)
                t2 = ttl.copy(b[0:2, 0:2], y)
                t1.wait()
                t2.wait()

        @ttl.datamovement()
        def w():
            with cbs[2].wait() as z:
                tx = ttl.copy(z, out[0:2, 0:2])
                tx.wait()

    with pytest.raises(Unsupported):
        tilewise.plan(_t(ttnn, (64, 64)), _t(ttnn, (64, 64)), _t(ttnn, (64, 64)))


def _simple_kernel(ttl, body_compute=None, read_shape=None, grid=(1, 1), buffer_factor=2, cb_shape=(1, 1)):
    @ttl.kernel(grid=grid)
    def k(a, out):
        a_cb = ttl.make_circular_buffer_like(a, shape=cb_shape, buffer_factor=buffer_factor)
        o_cb = ttl.make_circular_buffer_like(out, shape=cb_shape, buffer_factor=buffer_factor)

        @ttl.compute()
        def c():
            if body_compute is not None:
                body_compute(a_cb, o_cb)
                return
            with a_cb.wait() as x, o_cb.reserve() as y:
                y.store(x + x)

        @ttl.datamovement()
        def r():
            with a_cb.reserve() as x:
                sl = read_shape or (slice(0, cb_shape[0]), slice(0, cb_shape[1]))
                tx = ttl.copy(a[sl], x)
                tx.wait()

        @ttl.datamovement()
        def w():
            with o_cb.wait() as y:
                tx = ttl.copy(y, out[0:cb_shape[0], 0:cb_shape[1]])
                tx.wait()
    return k


def test_copy_shape_mismatch_message(tt):
    ttl, ttnn = tt
    k = _simple_kernel(ttl, read_shape=(slice(0, 2), slice(0, 1)))
    with pytest.raises(ValueError, match=r"does not match Block shape \(1, 1\) tiles"):
        k.plan(_t(ttnn, (64, 64)), _t(ttnn, (64, 64)))


def test_deadlock_is_reported(tt):
    from ttl_b200.trace import DeadlockError
    ttl, ttnn = tt

    def compute(a_cb, o_cb):
        with a_cb.wait() as x, o_cb.reserve() as y:
            y.store(x + x)
        with a_cb.wait() as x:      # nobody produces a second block
            pass

    k = _simple_kernel(ttl, body_compute=compute)
    with pytest.raises(DeadlockError, match="Deadlock detected"):
        k.plan(_t(ttnn, (32, 32)), _t(ttnn, (32, 32)))


def test_cb_contract_errors(tt):
    ttl, ttnn = tt

    def double_wait(a_cb, o_cb):
        a_cb.wait()
        a_cb.wait()

    with pytest.raises(RuntimeError, match=r"Cannot call wait\(\) again before pop\(\)"):
        _simple_kernel(ttl, body_compute=double_wait).plan(_t(ttnn, (32, 32)), _t(ttnn, (32, 32)))

    def read_unwritten(a_cb, o_cb):
        with a_cb.wait() as x, o_cb.reserve() as y:
            y.store(y + x)

    with pytest.raises(RuntimeError, match=r"must-write \(MW\) state"):
        _simple_kernel(ttl, body_compute=read_unwritten).plan(_t(ttnn, (32, 32)), _t(ttnn, (32, 32)))

    def index_block(a_cb, o_cb):
        with a_cb.wait() as x, o_cb.reserve() as y:
            y.store(x[0])

    with pytest.raises(RuntimeError, match="Block indexing"):
        _simple_kernel(ttl, body_compute=index_block).plan(_t(ttnn, (32, 32)), _t(ttnn, (32, 32)))

    def forgot_pop(a_cb, o_cb):
        x = a_cb.wait()
        with o_cb.reserve() as y:
            y.store(x + x)

    with pytest.raises(RuntimeError, match="incomplete CircularBuffer operations"):
        _simple_kernel(ttl, body_compute=forgot_pop).plan(_t(ttnn, (32, 32)), _t(ttnn, (32, 32)))


def test_cb_outside_kernel_and_bad_args(tt):
    ttl, ttnn = tt
    cb = ttl.make_circular_buffer_like(_t(ttnn, (32, 32)), shape=(1, 1))
    with pytest.raises(RuntimeError, match="created outside of a kernel context"):
        cb.reserve()
    with pytest.raises(ValueError, match="2-tuple"):
        ttl.make_circular_buffer_like(_t(ttnn, (32, 32)), shape=(1, 1, 1))
    with pytest.raises(ValueError, match="buffer_factor"):
        ttl.make_circular_buffer_like(_t(ttnn, (32, 32)), shape=(1, 1), buffer_factor=0)


def test_broadcast_validation(tt):
    ttl, ttnn = tt

    def bad_bcast(a_cb, o_cb):
        with a_cb.wait() as x, o_cb.reserve() as y:
            y.store(ttl.math.broadcast(x, dims=[0]) + x)

    k = _simple_kernel(ttl, body_compute=bad_bcast, cb_shape=(2, 1))
    with pytest.raises(ValueError, match="dimension must have size 1"):
        k.plan(_t(ttnn, (64, 32)), _t(ttnn, (64, 32)))

    def no_dims(a_cb, o_cb):
        with a_cb.wait() as x, o_cb.reserve() as y:
            y.store(ttl.math.broadcast(x) + x)

    with pytest.raises(ValueError, match="dims parameter is required"):
        _simple_kernel(ttl, body_compute=no_dims).plan(_t(ttnn, (32, 32)), _t(ttnn, (32, 32)))


def test_kernel_needs_three_threads(tt):
    ttl, ttnn = tt

    @ttl.kernel(grid=(1, 1))
    def k(a):
        @ttl.compute()
        def c():
            pass

    with pytest.raises(ValueError, match="exactly 3 threads"):
        k.plan(_t(ttnn, (32, 32)))


def test_core_and_grid_size_follow_the_simulator(tt):
    from ttl_b200 import trace
    assert trace.grid_size_of((8, 8), 1) == 64
    assert trace.grid_size_of((8, 8), 3) == (8, 8, 1)
    assert trace.grid_size_of((2, 3, 4), 2) == (2, 12)
    assert trace.core_coords(19, (8, 8), 2) == (2, 3)
    assert trace.core_coords(19, (8, 8), 1) == 19
    assert trace.core_coords(5, (2, 3), 3) == (1, 2, 0)
    assert trace.flatten_core_index((2, 3), (8, 8)) == 19


def test_split_work_to_cores(tt):
    ttl, ttnn = tt
    n, all_c, g1, g2, u1, u2 = ttnn.split_work_to_cores(ttnn.CoreCoord(8, 8), 100, row_wise=True)
    assert (n, g1.num_cores(), g2.num_cores(), u1, u2) == (64, 36, 28, 2, 1)
    assert g1.ranges()[1].start == ttnn.CoreCoord(1, 0)          # row-wise: x fastest
    n, _, g1, g2, u1, u2 = ttnn.split_work_to_cores(ttnn.CoreCoord(13, 10), 64)
    assert (n, g1.num_cores(), g2.num_cores(), u1, u2) == (64, 64, 0, 1, 0)
    assert ttnn.split_work_to_cores(ttnn.CoreCoord(2, 2), 0)[0] == 0


def test_overlapping_writes_rejected(tt):
    from ttl_b200 import Unsupported
    ttl, ttnn = tt

    @ttl.kernel(grid=(2, 1))
    def k(a, out):
        a_cb = ttl.make_circular_buffer_like(a, shape=(1, 1))
        o_cb = ttl.make_circular_buffer_like(out, shape=(1, 1))

        @ttl.compute()
        def c():
            with a_cb.wait() as x, o_cb.reserve() as y:
                y.store(x)

        @ttl.datamovement()
        def r():
            with a_cb.reserve() as x:
                tx = ttl.copy(a[0, ttl.core(dims=1) if distinct else 0], x)
                tx.wait()

        @ttl.datamovement()
        def w():
            with o_cb.wait() as y:
                tx = ttl.copy(y, out[0, 0])   # both cores write tile (0, 0)
                tx.wait()

    distinct = True     # the two cores write different values to the same tile: order-dependent
    with pytest.raises(Unsupported, match="written more than once"):
        k.plan(_t(ttnn, (32, 64)), _t(ttnn, (32, 32)))
    distinct = False    # every core writes the same value (a program that ignores the grid): one write
    d = k.plan(_t(ttnn, (32, 64)), _t(ttnn, (32, 32), torch.bfloat16)).describe()
    assert len(d) == 1 and d[0]["rect_tiles"] == (0, 1, 0, 1)


def test_merge_rects():
    from ttl_b200.recognize import merge_rects
    rects = [(r, r + 2, c, c + 1) for c in range(4) for r in range(0, 8, 2)]
    assert merge_rects(rects) == [(0, 8, 0, 4)]
    assert merge_rects([(0, 1, 0, 1), (1, 2, 1, 2)]) == [(0, 1, 0, 1), (1, 2, 1, 2)]
    assert merge_rects([]) == []


def test_launch_without_gpu_fails_loudly(backend, tt):
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from ttl_b200 import BackendError
    _, mods = backend
    ttl, ttnn = tt
    a, b, o = (_t(ttnn, (64, 64)) for _ in range(3))
    with pytest.raises(BackendError, match="no CPU fallback"):
        mods["eltwise"].eltwise_add(a, b, o)


def test_every_case_program_is_recognised(backend, tt):
    _, mods = backend
    ttl, ttnn = tt
    for case in cases.CASES + cases.MATMUL_CASES:
        ins = [ttnn.from_torch(t) for t in case.make_inputs()]
        out = _t(ttnn, case.out_shape, case.dtype)
        plan = case.get_program(mods, f32acc=(case.mode == "f32")).plan(*ins, out)
        kinds = {d["kind"] for d in plan.describe()}
        assert kinds == ({"matmul_bf16"} if case.module == "matmul" else {"eltwise"}), case.name


def test_translate_prints_plan_and_cuda_source(tmp_path):
    """ttlang-b200-translate on a small program file: launch plan + specialised CUDA source, no GPU."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    prog = tmp_path / "prog.py"
    prog.write_text(
        "import sys; sys.path.insert(0, %r)\n"
        "import importlib.util, torch, ttnn\n"
        "spec = importlib.util.spec_from_file_location('pe', %r); m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)\n"
        "z = lambda s: ttnn.from_torch(torch.zeros(s, dtype=torch.bfloat16))\n"
        "m.fused_exp_bcast_f32acc(z((128, 256)), z((1, 1)), z((1, 256)), z((128, 256)), z((128, 256)))\n"
        % (str(root / "tests"), str(root / "tests" / "programs" / "eltwise.py")))
    r = subprocess.run([sys.executable, "-m", "ttl_b200.translate", str(prog)], capture_output=True, text=True,
                       cwd=root, env={**__import__("os").environ, "PYTHONPATH": str(root / "tt-lang_b200")}, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert '"kind": "eltwise"' in r.stdout and "ttlb_eltwise_jit" in r.stdout and "expf(a)" in r.stdout


def test_translate_prints_reduction_and_row_fused_sources(tmp_path):
    """ttlang-b200-translate on programs with reductions: the generated reduction kernel and the row-resident kernel."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    prog = tmp_path / "prog.py"
    prog.write_text(
        "import importlib.util, torch, ttnn\n"
        "spec = importlib.util.spec_from_file_location('pr', %r); m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)\n"
        "z = lambda s: ttnn.from_torch(torch.zeros(s, dtype=torch.bfloat16))\n"
        "m.make_reduce('sum', [0])(z((128, 256)), z((32, 32)), z((1, 256)))\n"
        "m.make_softmax()(z((128, 256)), z((32, 32)), z((128, 256)))\n"
        % str(root / "tests" / "programs" / "reduce.py"))
    r = subprocess.run([sys.executable, "-m", "ttl_b200.translate", str(prog)], capture_output=True, text=True,
                       cwd=root, env={**__import__("os").environ, "PYTHONPATH": str(root / "tt-lang_b200")}, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert '"kind": "reduce_sum"' in r.stdout and "ttlb_reduce_jit" in r.stdout
    assert '"kind": "row_fused"' in r.stdout and "ttlb_rowfused_jit" in r.stdout and "source unavailable" not in r.stdout


def _shift_program():
    import ttl

    @ttl.kernel(grid=(1, 1))
    def shift(t, b):
        t_cb = ttl.make_circular_buffer_like(t, shape=(1, 1), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(t, shape=(1, 1), buffer_factor=2)

        @ttl.compute()
        def comp():
            for _ in range(2):
                with t_cb.wait() as x, b_cb.wait() as y, o_cb.reserve() as o:
                    o.store(x + y)

        @ttl.datamovement()
        def rd():
            for i in range(2):
                with t_cb.reserve() as x, b_cb.reserve() as y:
                    ttl.copy(t[i, 0], x).wait()
                    ttl.copy(b[i, 0], y).wait()

        @ttl.datamovement()
        def wr():
            for i in range(2):
                with o_cb.wait() as o:
                    ttl.copy(o, t[i + 1, 0]).wait()

    return shift


def test_program_that_reads_tiles_it_also_writes_is_refused(backend):
    """t[i+1] = t[i] + b: every launch of a plan runs in parallel, so a program whose result depends on the order
    of its own writes and reads is refused instead of being turned into a racing launch; updating a tensor in
    place, tile for tile, is fine."""
    import torch
    import ttl
    import ttnn
    from ttl_b200 import Unsupported
    t = ttnn.Tensor(torch.zeros(96, 32, dtype=torch.bfloat16))
    b = ttnn.Tensor(torch.zeros(64, 32, dtype=torch.bfloat16))
    with pytest.raises(Unsupported, match="also writes"):
        _shift_program().plan(t, b)

    @ttl.kernel(grid=(1, 1))
    def in_place(t, b):
        t_cb = ttl.make_circular_buffer_like(t, shape=(1, 1), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(t, shape=(1, 1), buffer_factor=2)

        @ttl.compute()
        def comp():
            for _ in range(2):
                with t_cb.wait() as x, b_cb.wait() as y, o_cb.reserve() as o:
                    o.store(x + y)

        @ttl.datamovement()
        def rd():
            for i in range(2):
                with t_cb.reserve() as x, b_cb.reserve() as y:
                    ttl.copy(t[i, 0], x).wait()
                    ttl.copy(b[i, 0], y).wait()

        @ttl.datamovement()
        def wr():
            for i in range(2):
                with o_cb.wait() as o:
                    ttl.copy(o, t[i, 0]).wait()

    d = in_place.plan(ttnn.Tensor(torch.zeros(64, 32, dtype=torch.bfloat16)), b).describe()
    assert len(d) == 1 and d[0]["kind"] == "eltwise" and d[0]["out"] == 0 and d[0]["inputs"][0][:1] == (0,)


def test_matmul_whose_operand_is_its_output_is_refused(backend):
    import torch
    import ttnn
    from ttl_b200 import Unsupported
    _, mods = backend
    a = ttnn.Tensor(torch.zeros(64, 64, dtype=torch.bfloat16))
    b = ttnn.Tensor(torch.zeros(64, 64, dtype=torch.bfloat16))
    with pytest.raises(Unsupported, match="also writes"):
        mods["matmul"].singlecore_matmul.plan(a, b, a)

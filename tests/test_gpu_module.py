"""The code-object half of the device FFI: a kernel of the library loaded from its stand-alone cubin by
name and launched with the kernelParams ABI must give the bits of the linked entry point
(crates/v4flash-hip/src/module.rs:28-57,141-171 in the reference); stream memory operations order two
streams at execution time (sys.rs:290-302, het/forward_layer.rs:436-449)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_module_load_get_function_launch_matches_linked_kernel():
    import torch
    from deepstrix_b200 import _build, moe
    torch.cuda.set_device(0)
    T, k, H = 37, 6, 2048
    rng = np.random.default_rng(12)
    partial = torch.from_numpy(rng.standard_normal((T * k + T, H)).astype(np.float32)).cuda()
    want = moe.reduce_partials(partial, T, k, with_shared=True)
    # the operator itself against a plain restatement: slot-order f32 adds from 0, then the shared row
    acc = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    for s in range(k):
        acc = acc + partial[:T * k].view(T, k, H)[:, s]
    acc = acc + partial[T * k:]
    assert torch.equal(want, acc.to(torch.bfloat16))
    mod = moe.Module(open(_build.CUBIN_PATH, "rb").read())
    fn = mod.get_function("dsx_combine_kernel")
    assert mod.get_function("dsx_combine_kernel").value == fn.value      # second lookup: the module's name table
    with pytest.raises(moe.DsxError):
        mod.get_function("no_such_kernel")
    out = torch.zeros((T, H), dtype=torch.bfloat16, device="cuda")
    n = T * (H // 4)
    args = [C.c_void_p(partial.data_ptr()), C.c_int64(T), C.c_int(k), C.c_int64(H), C.c_int(1), C.c_void_p(0), C.c_int(0), C.c_int(0),
            C.c_void_p(out.data_ptr()), C.c_void_p(0)]              # ..., out, out_rows (no row table)
    before = moe.launch_count()
    moe.Module.launch_raw(fn, ((n + 255) // 256, 1, 1), (256, 1, 1), 0, args)
    torch.cuda.synchronize()
    assert moe.launch_count() == before + 1                               # the launch audit counts raw launches too
    assert torch.equal(out, want)
    with pytest.raises(moe.DsxError):
        moe.Module(b"this is not a code object")
    mod.close()


def test_stream_value_ops_order_two_streams():
    import torch
    from deepstrix_b200 import moe
    torch.cuda.set_device(0)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    data = torch.zeros(1024, dtype=torch.float32, device="cuda")
    result = torch.zeros(1024, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    producer, consumer = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(consumer):           # issued FIRST: waits, on the device, until the flag reaches 7
        moe.stream_wait_value32(flag.data_ptr(), 7, flags=0)
        result.copy_(data)
    with torch.cuda.stream(producer):
        data.fill_(3.0)
        moe.stream_write_value32(flag.data_ptr(), 7)
    torch.cuda.synchronize()
    assert int(flag.item()) == 7
    assert bool((result == 3.0).all())


def test_graph_kernel_node_set_params_repoints_a_captured_launch():
    """A launch captured into a graph, instantiated once, then pointed at other buffers without re-capturing
    (hipGraphExecKernelNodeSetParams in the reference, crates/v4flash-hip/src/sys.rs:372)."""
    import torch
    from deepstrix_b200 import _build, moe
    torch.cuda.set_device(0)
    lib = moe.lib()
    T, k, H = 9, 4, 1024
    rng = np.random.default_rng(3)
    parts = [torch.from_numpy(rng.standard_normal((T * k + T, H)).astype(np.float32)).cuda() for _ in range(2)]
    outs = [torch.zeros((T, H), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    want = [moe.reduce_partials(p, T, k, with_shared=True) for p in parts]
    mod = moe.Module(open(_build.CUBIN_PATH, "rb").read())
    fn = mod.get_function("dsx_combine_kernel")
    n = T * (H // 4)

    def args_for(i):
        return [C.c_void_p(parts[i].data_ptr()), C.c_int64(T), C.c_int(k), C.c_int64(H), C.c_int(1), C.c_void_p(0), C.c_int(0), C.c_int(0),
                C.c_void_p(outs[i].data_ptr()), C.c_void_p(0)]       # ..., out, out_rows (no row table)
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        moe._check(lib.dsx_graph_begin_capture(C.c_void_p(stream.cuda_stream)))
        moe.Module.launch_raw(fn, ((n + 255) // 256, 1, 1), (256, 1, 1), 0, args_for(0))
        ge, g = C.c_void_p(), C.c_void_p()
        moe._check(lib.dsx_graph_end_capture_keep(C.c_void_p(stream.cuda_stream), C.byref(ge), C.byref(g)))
        count = C.c_size_t(0)
        moe._check(lib.dsx_graph_kernel_nodes(g, None, C.byref(count)))
        assert count.value == 1
        nodes = (C.c_void_p * 1)()
        moe._check(lib.dsx_graph_kernel_nodes(g, nodes, C.byref(count)))
        moe._check(lib.dsx_graph_launch(ge, C.c_void_p(stream.cuda_stream)))
        stream.synchronize()
        assert torch.equal(outs[0], want[0]) and not bool(outs[1].any())
        a1 = args_for(1)
        ptrs = (C.c_void_p * len(a1))(*[C.cast(C.pointer(a), C.c_void_p) for a in a1])
        moe._check(lib.dsx_graph_exec_kernel_node_set_params(ge, nodes[0], None, None, None, 0, ptrs))
        moe._check(lib.dsx_graph_launch(ge, C.c_void_p(stream.cuda_stream)))
        stream.synchronize()
        assert torch.equal(outs[1], want[1])
        lib.dsx_graph_destroy(ge)
        lib.dsx_graph_template_destroy(g)
    mod.close()

"""rtxb_mxfp8_linear_fwd_noalloc — the forward for callers that cannot allocate.

Hosts that only own the input and output buffers they were handed (a generated
wrapper, a plugin inside someone else's memory pool, a section where cudaMalloc
may not run) have no workspace to pass.  This entry point keeps the quantized
operands in a fixed 32 MiB array inside the library instead.  The test drives it
through the C ABI exactly as such a host would — three pointers, the sizes, a
stream — and requires the same output bits as the workspace-taking entry point,
on two calls in a row that share the array.  It lives in the last-collected test
file so that a run stopping at the first failure has already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(native_lib):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from rtx_b200 import _native as N
    from rtx_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    return N, ops, dev


def _noalloc(N, ops, x, w, dev):
    m, k = x.shape
    n = w.shape[0]
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    before = torch.cuda.memory_allocated(dev)
    N.call("rtxb_mxfp8_linear_fwd_noalloc", x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, N.ROUND_INFINITY,
           torch.cuda.current_stream().cuda_stream, ops.status_word(dev).data_ptr())
    assert torch.cuda.memory_allocated(dev) == before   # torch's allocator was not involved either
    return out


def test_noalloc_forward_matches_workspace_forward_twice(env):
    N, ops, dev = env
    ws = ops.Workspace(dev)
    # two different problems back to back: the second call finds the first one's operands in the array
    for seed, (m, n, k) in ((21, (300, 700, 1000)), (22, (129, 257, 96))):
        torch.manual_seed(seed)
        x = torch.randn(m, k).bfloat16().to(dev)
        w = (torch.randn(n, k) / k ** 0.5).bfloat16().to(dev)
        want = ops.mxfp8_linear_fwd(x, w, ws)
        got = _noalloc(N, ops, x, w, dev)
        torch.cuda.synchronize()
        ops.check_device_status(dev)
        assert not torch.isnan(got.float()).any()
        # same kernels, same operand bytes: the tests' bar for this path is bit equality
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    # and once more with the first shape, now over the second call's leftovers
    torch.manual_seed(21)
    x = torch.randn(300, 1000).bfloat16().to(dev)
    w = (torch.randn(700, 1000) / 1000 ** 0.5).bfloat16().to(dev)
    assert torch.equal(_noalloc(N, ops, x, w, dev), ops.mxfp8_linear_fwd(x, w, ws))
    torch.cuda.synchronize()
    ops.check_device_status(dev)


def test_noalloc_refuses_shapes_beyond_its_array(env):
    N, ops, dev = env
    m, n, k = 8192, 8192, 4096   # needs ~69 MB of quantized operands: more than the 32 MiB array
    assert N.query("rtxb_mxfp8_linear_workspace_bytes", m, n, k) > N.NOALLOC_SCRATCH_BYTES
    x = torch.zeros(1, dtype=torch.bfloat16, device=dev)   # never dereferenced: the call must refuse first
    code = N.load().rtxb_mxfp8_linear_fwd_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), m, n, k, 1, None, None)
    assert code == N.E_SCRATCH_CAPACITY
    # the refusal says how much the shape needs and how much the array holds
    with pytest.raises(N.NativeError, match=r"built-in scratch array.*needs \d+ bytes.*holds 33554432"):
        N.check(code, "rtxb_mxfp8_linear_fwd_noalloc")
    torch.cuda.synchronize()


def test_noalloc_refuses_a_stream_of_another_device(env):
    """The array's address is looked up for the current device, so a stream that lives on a different GPU is
    refused before anything is launched.  Needs two GPUs (skipped otherwise)."""
    N, ops, dev = env
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(128, 128, dtype=torch.bfloat16, device=dev)     # real buffers of the right sizes all the same
    other = torch.cuda.Stream(device=torch.device("cuda", 1))
    code = N.load().rtxb_mxfp8_linear_fwd_noalloc(x.data_ptr(), w.data_ptr(), out.data_ptr(), 128, 128, 64, 1,
                                                  other.cuda_stream, None)
    assert code == -1
    with pytest.raises(N.NativeError, match="stream belongs to device 1"):
        N.check(code, "rtxb_mxfp8_linear_fwd_noalloc")
    torch.cuda.synchronize()

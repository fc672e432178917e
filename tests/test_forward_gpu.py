"""Forward parity on the GPU: the CUDA kernels (through the public `ddf` op and
hence the C ABI) against the float64 CPU oracle on identical seeded inputs."""
import pytest
import torch

from tests.util import DTYPES, check_close, make_inputs, oracle_forward

pytestmark = pytest.mark.gpu


def _lib():
    from ddfnet_b200 import _lib
    return _lib


def _run(x, cf, sf, k, d, s, m, version=""):
    from ddfnet_b200 import ddf
    dev = torch.device("cuda:0")
    return ddf(x.to(dev), cf.to(dev), sf.to(dev), k, d, s, m, version)


def _no_fault():
    assert _lib().load().ddf_b200_take_fault() == 0


# ------------------------------------------------------------------ generic kernel: wide sweep
GENERIC = []
for k, d in [(1, 1), (3, 1), (3, 2), (3, 3), (5, 1), (5, 2), (7, 1)]:
    for s in (1, 2):
        GENERIC.append((2, 3, 9, 11, k, d, s))
GENERIC += [(1, 1, 5, 5, 3, 1, 1), (1, 33, 10, 12, 3, 1, 2), (1, 70, 10, 10, 3, 2, 1),
            (3, 8, 7, 7, 3, 1, 1), (2, 5, 13, 9, 5, 2, 2), (1, 2, 4, 30, 3, 1, 3)]


@pytest.mark.parametrize("shape", GENERIC)
@pytest.mark.parametrize("dt", ["f32", "f64", "f16", "bf16"])
def test_generic_forward(shape, dt):
    B, C, H, W, k, d, s = shape
    dtype = DTYPES[dt]
    x, cf, sf = make_inputs(B, C, H, W, k, s, dtype, seed=100 + k * 10 + d + s, with_go=False)
    for m in ("mul", "add"):
        out = _run(x, cf, sf, k, d, s, m, "o")
        assert out.dtype == dtype and out.shape == (B, C, H // s, W // s)
        check_close(out, oracle_forward(x, cf, sf, k, d, s, m), dtype, f"generic {shape} {dt} {m}")


# ------------------------------------------------------------------ streaming kernel
# B, C, H, W, k, d, s -- every (k, d, s, P) instantiation, plane runs that cross
# sample boundaries inside a CTA, several samples inside one stage (small C),
# fewer plane groups than SMs, and widths for each pixels-per-thread choice.
STREAM = [
    (4, 16, 56, 56, 3, 1, 1),    # P = 8
    (3, 64, 28, 28, 3, 1, 1),    # P = 4, two planes per pass
    (8, 32, 14, 14, 3, 1, 1),    # P = 2
    (8, 64, 7, 7, 3, 1, 1),      # P = 1 (sub-word path for 2-byte types)
    (40, 8, 7, 7, 3, 1, 1),      # C = planes per pass: a new sample every pass
    (300, 2, 14, 14, 3, 1, 1),   # more samples than CTAs, two planes per sample
    (3, 32, 56, 56, 3, 1, 2),    # stride 2, P = 4
    (8, 32, 28, 28, 3, 1, 2),    # stride 2, P = 2
    (8, 64, 14, 14, 3, 1, 2),    # stride 2, P = 1
    (2, 16, 57, 56, 3, 1, 2),    # odd height at stride 2 (floor output size)
    (3, 16, 56, 56, 3, 2, 1),    # dilation 2, P = 8
    (3, 32, 28, 28, 3, 2, 1),
    (8, 32, 14, 14, 3, 2, 1),
    (3, 32, 28, 28, 5, 1, 1),    # k = 5
    (8, 32, 14, 14, 5, 1, 1),
    (3, 32, 28, 28, 5, 2, 1),
    (2, 24, 20, 24, 3, 1, 1),    # non-square, H*W/8 = 60 tasks, 6 planes per pass
    (1, 8, 40, 64, 3, 1, 1),     # wide plane, single sample
    (2, 16, 16, 8, 3, 1, 1),
    (2, 64, 56, 56, 3, 1, 1),    # plane-ring kernel (2-byte types): one plane per pass
    (5, 24, 28, 28, 3, 1, 1),    # plane-ring: three planes per pass, run crossing samples
    (3, 48, 14, 14, 3, 1, 1),    # plane-ring: sixteen planes per pass
    (5, 40, 28, 28, 3, 1, 2),    # plane-ring, stride 2
    (2, 8, 57, 56, 3, 1, 1),     # 56 wide but 57 high: ring kernel with a non-square plane
    (3, 128, 7, 7, 3, 1, 1),     # row kernel (2-byte types): two chunks per sample
    (400, 64, 7, 7, 3, 1, 1),    # row kernel: a new sample every chunk, both filter buffers reused
    (2400, 64, 7, 7, 3, 1, 1),   # row kernel: more chunks per CTA than ring slots
    (3, 192, 14, 14, 3, 1, 2),   # row kernel, stride 2
    (1100, 64, 14, 14, 3, 1, 2), # row kernel, stride 2: ring slots reused
    (5, 96, 14, 14, 3, 1, 1),    # row kernel, 14-pixel rows: three chunks per sample
    (2100, 32, 14, 14, 3, 1, 1), # row kernel, 14-pixel rows: ring slots and filter buffers reused
    (300, 8, 28, 28, 3, 1, 1),   # row kernel, two 14-pixel segments per row, one chunk per sample
    (40, 6, 56, 56, 3, 1, 1),    # row kernel, four segments per row, three chunks per sample
    (600, 32, 28, 28, 3, 1, 2),  # row kernel, stride 2, two 7-pixel segments per row: slots reused
    (320, 16, 56, 56, 3, 1, 2),  # row kernel, stride 2, four segments per row: slots reused
]


@pytest.mark.parametrize("shape", STREAM)
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_stream_forward(shape, dt):
    B, C, H, W, k, d, s = shape
    dtype = DTYPES[dt]
    x, cf, sf = make_inputs(B, C, H, W, k, s, dtype, seed=200 + H + k + d + s, with_go=False)
    for m in ("mul", "add"):
        out = _run(x, cf, sf, k, d, s, m, "f")
        check_close(out, oracle_forward(x, cf, sf, k, d, s, m), dtype, f"stream {shape} {dt} {m}")
    _no_fault()


@pytest.mark.parametrize("shape", [(2100, 32, 14, 14, 3, 1, 1), (300, 8, 28, 28, 3, 1, 1), (400, 64, 7, 7, 3, 1, 1),
                                   (4800, 64, 7, 7, 3, 1, 1), (320, 16, 56, 56, 3, 1, 2), (96, 64, 56, 56, 3, 1, 1)])
@pytest.mark.parametrize("mode", ["mul", "add"])
def test_results_do_not_change_between_runs(shape, mode):
    """A new sample every chunk makes the kernel recycle its two spatial-filter buffers as fast
    as it can, and the last three shapes give every CTA several times more chunks than ring
    slots; a value read after its buffer was handed back shows up as a run-to-run difference
    (the kernels have no atomics: equal inputs must give equal bits)."""
    B, C, H, W, k, d, s = shape
    dev = torch.device("cuda:0")
    x, cf, sf = [t.to(dev) for t in make_inputs(B, C, H, W, k, s, torch.bfloat16, seed=5, with_go=False)]
    from ddfnet_b200 import ddf
    ref = ddf(x, cf, sf, k, d, s, mode, "f")
    for _ in range(40):
        assert torch.equal(ddf(x, cf, sf, k, d, s, mode, "f"), ref)
    _no_fault()


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("mode", ["mul", "add"])
def test_gradients_do_not_change_between_runs(dt, mode):
    """The same for the backward: grad-x runs in the row kernel with the spatial-filter registers
    gathered from a recycled buffer, and the two filter gradients are summed in a fixed order."""
    from ddfnet_b200 import ddf
    dev = torch.device("cuda:0")
    B, C, H = 300, 8, 28
    x, cf, sf, go = [t.to(dev) for t in make_inputs(B, C, H, H, 3, 1, DTYPES[dt], seed=6)]
    def grads():
        xs = [t.detach().requires_grad_() for t in (x, cf, sf)]
        ddf(*xs, 3, 1, 1, mode).backward(go)
        return [t.grad for t in xs]
    ref = grads()
    for _ in range(20):
        for a, b in zip(grads(), ref):
            assert torch.equal(a, b)
    _no_fault()


RAGGED = [(5, 32, 14, 14), (12, 32, 14, 14), (5, 64, 7, 7), (12, 64, 7, 7), (3, 24, 14, 14), (7, 8, 7, 7)]


@pytest.mark.parametrize("shape", RAGGED)
@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
def test_streaming_kernels_take_ragged_sizes(shape, dt):
    """Batch sizes whose tensors are not multiples of 16 bytes (every B that is not a multiple
    of 8 at 7x7, every odd B at 14x14 in the 2-byte types): the bulk copies stop at the
    tensor's last whole 16 bytes and the rest is fetched with plain loads, so the streaming
    kernels serve them ('f') -- also when the tensors sit at the very end of an allocation."""
    B, C, H, W = shape
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    x, cf, sf = make_inputs(B, C, H, W, 3, 1, dtype, seed=300 + B + H, with_go=False)

    def at_end(t):   # a view that ends exactly at the end of its own allocation
        flat = torch.empty(t.numel() + 128, dtype=t.dtype, device=dev)
        v = flat[128:].view(t.shape)
        v.copy_(t)
        return v

    from ddfnet_b200 import ddf
    for m in ("mul", "add"):
        out = ddf(at_end(x), at_end(cf), at_end(sf), 3, 1, 1, m, "f")
        check_close(out, oracle_forward(x, cf, sf, 3, 1, 1, m), dtype, f"ragged {shape} {dt} {m}")
    _no_fault()


def test_wait_limit_reports_a_fault_and_the_context_survives(monkeypatch):
    """A bounded wait that runs out: every stage is announced 16 bytes larger than what is
    copied, so no stage ever completes; with a limit of about a millisecond the compute warps
    give up, the kernel returns, the fault word reads 1 (a compute warp gave up waiting for a
    stage) and the next ordinary call works."""
    lib = _lib()
    L = lib.load()
    dev = torch.device("cuda:0")
    B, C, H = 8, 64, 28
    x, cf, sf = (t.to(dev) for t in make_inputs(B, C, H, H, 3, 1, torch.bfloat16, 77, with_go=False))
    out = torch.empty_like(x)
    stream = torch.cuda.current_stream().cuda_stream
    args = (x.data_ptr(), cf.data_ptr(), sf.data_ptr(), out.data_ptr(), B, C, H, H, 3, 1, 1, lib.MUL, lib.BF16)
    assert L.ddf_b200_take_fault() == 0
    assert L.ddf_b200_forward_waitlimit(*args, 2_000_000, 1, stream) == 0
    assert L.ddf_b200_take_fault() == 1
    assert L.ddf_b200_take_fault() == 0          # reading the word clears it
    # the same entry point without starvation is an ordinary forward
    assert L.ddf_b200_forward_waitlimit(*args, 2_000_000_000, 0, stream) == 0
    want = oracle_forward(x.cpu(), cf.cpu(), sf.cpu(), 3, 1, 1, "mul")
    check_close(out, want, torch.bfloat16, "after a starved launch")
    check_close(_run(x, cf, sf, 3, 1, 1, "mul"), want, torch.bfloat16, "ordinary call after a starved launch")
    _no_fault()
    # the Python mirror's debug mode (DDF_B200_DEBUG=1) turns a recorded fault into an exception
    monkeypatch.setattr(lib, "_DEBUG", True)
    with pytest.raises(RuntimeError, match="bounded wait ran out"):
        lib.check(L.ddf_b200_forward_waitlimit(*args, 2_000_000, 1, stream))
    monkeypatch.setattr(lib, "_DEBUG", False)
    _no_fault()
    # shapes outside the ring kernel's set are refused, not run
    xf = x.float()
    assert L.ddf_b200_forward_waitlimit(xf.data_ptr(), cf.float().data_ptr(), sf.float().data_ptr(),
                                        torch.empty_like(xf).data_ptr(), B, C, H, H, 3, 1, 1, lib.MUL, lib.F32,
                                        2_000_000, 0, stream) == -7


def test_stream_rejects_what_it_cannot_do():
    from ddfnet_b200._lib import DDFError
    x, cf, sf = make_inputs(1, 3, 9, 11, 7, 1, torch.float32, seed=1, with_go=False)
    with pytest.raises(DDFError):
        _run(x, cf, sf, 7, 1, 1, "mul", "f")


def test_stream_writes_only_its_output():
    """Canaries either side of the output buffer stay intact."""
    from ddfnet_b200 import _lib
    L = _lib.load()
    dev = torch.device("cuda:0")
    B, C, H, W = 3, 32, 28, 28
    x, cf, sf = (t.to(dev) for t in make_inputs(B, C, H, W, 3, 1, torch.bfloat16, 5, with_go=False))
    n = B * C * H * W
    pad = 4096
    buf = torch.full((n + 2 * pad,), 7.0, dtype=torch.bfloat16, device=dev)
    out = buf[pad:pad + n]
    for variant in (_lib.VARIANT_GENERIC, _lib.VARIANT_STREAM):
        buf.fill_(7.0)
        rc = L.ddf_b200_forward(x.data_ptr(), cf.data_ptr(), sf.data_ptr(), out.data_ptr(),
                                B, C, H, W, 3, 1, 1, _lib.MUL, _lib.BF16, variant,
                                torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert (buf[:pad] == 7.0).all() and (buf[pad + n:] == 7.0).all()
        check_close(out.view(B, C, H, W), oracle_forward(x.cpu(), cf.cpu(), sf.cpu(), 3, 1, 1, "mul"),
                    torch.bfloat16, "canary case")
    _no_fault()


# ------------------------------------------------------------------ the benchmark configurations
def test_config1_fp32():
    # single op, mul, float32: B=2, C=64, 56x56, k=3
    x, cf, sf = make_inputs(2, 64, 56, 56, 3, 1, torch.float32, seed=1000, with_go=False)
    want = oracle_forward(x, cf, sf, 3, 1, 1, "mul")
    for ver in ("", "o", "f"):
        check_close(_run(x, cf, sf, 3, 1, 1, "mul", ver), want, torch.float32, f"config 1 '{ver}'")
    _no_fault()


CONFIG2 = [(64, 56, 1), (128, 28, 1), (256, 14, 1), (512, 7, 1), (128, 56, 2), (256, 28, 2), (512, 14, 2)]


@pytest.mark.parametrize("case", CONFIG2)
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_config2_full_size(case, dt):
    """ResNet-50 stage shapes at B = 128: the default kernel choice must be the
    streaming kernel and must match the oracle; doubling the input doubles the
    output exactly (a power-of-two scale commutes with every rounding)."""
    C, H, s = case
    B = 128
    dtype = DTYPES[dt]
    L = _lib().load()
    assert L.ddf_b200_plan(B, C, H, H, 3, 1, s, 0, {"bf16": 2, "f16": 1}[dt], 0) == _lib().VARIANT_STREAM
    x, cf, sf = make_inputs(B, C, H, H, 3, s, dtype, seed=2000 + C + s, with_go=False)
    for m in ("mul", "add"):
        out = _run(x, cf, sf, 3, 1, s, m)
        check_close(out, oracle_forward(x, cf, sf, 3, 1, s, m), dtype, f"config 2 {case} {dt} {m}")
        out2 = _run(x * 2, cf, sf, 3, 1, s, m)
        if dtype == torch.float16:   # float16 results below 2**-14 are subnormal: not scale-exact
            keep = out.abs() > 1e-3
            assert torch.equal(out2[keep], (out * 2)[keep])
        else:
            assert torch.equal(out2, out * 2)
    _no_fault()


# ------------------------------------------------------------------ interface behaviour
def test_interface_errors():
    from ddfnet_b200 import ddf
    dev = torch.device("cuda:0")
    x, cf, sf = (t.to(dev) for t in make_inputs(2, 4, 8, 8, 3, 1, torch.float32, 3, with_go=False))
    with pytest.raises(AssertionError):
        ddf(x.cpu(), cf, sf, 3, 1, 1, "mul")
    with pytest.raises(AssertionError):
        ddf(x, cf[:, :3], sf, 3, 1, 1, "mul")
    with pytest.raises(AssertionError):
        ddf(x, cf, sf[:, :8], 3, 1, 1, "mul")
    with pytest.raises(AssertionError):
        ddf(x, cf, sf, 3, 1, 1, "max")
    with pytest.raises(AssertionError):
        ddf(x, cf, sf, 4, 1, 1, "mul")
    with pytest.raises(RuntimeError):
        ddf(x.transpose(2, 3), cf, sf, 3, 1, 1, "mul")
    # mixed precision promotes, as the reference's float16 up-cast does
    out = ddf(x.half(), cf, sf, 3, 1, 1, "mul")
    assert out.dtype == torch.float32
    # 7 positional arguments, as DDFPack calls it
    assert ddf(x, cf, sf, 3, 1, 1, "add").shape == x.shape


def test_runs_on_the_callers_stream():
    from ddfnet_b200 import ddf
    dev = torch.device("cuda:0")
    x, cf, sf = (t.to(dev) for t in make_inputs(4, 64, 28, 28, 3, 1, torch.float16, 9, with_go=False))
    want = oracle_forward(x.cpu(), cf.cpu(), sf.cpu(), 3, 1, 1, "mul")
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        out = ddf(x, cf, sf, 3, 1, 1, "mul", "f")
    st.synchronize()
    check_close(out, want, torch.float16, "side stream")


def test_host_buffers_sync_and_async_paths():
    """ddf_host / ddf_host_async (pinned host tensors in, pinned host tensor out, chunks over
    rotating streams) against the oracle; several asynchronous calls in flight at once."""
    from ddfnet_b200.host import ddf_host, ddf_host_async
    dtype = torch.bfloat16
    cases = []
    for i, (B, C, H, s) in enumerate([(64, 64, 56, 1), (32, 128, 28, 2), (48, 256, 14, 1)]):
        x, cf, sf = make_inputs(B, C, H, H, 3, s, dtype, 900 + i, with_go=False)
        cases.append((x.pin_memory(), cf.pin_memory(), sf.pin_memory(), s))
    handles = [ddf_host_async(x, cf, sf, 3, 1, s, "mul", chunks=3) for (x, cf, sf, s) in cases]
    for (x, cf, sf, s), h in zip(cases, handles):
        out = h.wait()
        assert out.is_pinned() and not out.is_cuda
        check_close(out, oracle_forward(x, cf, sf, 3, 1, s, "mul"), dtype, "ddf_host_async")
    x, cf, sf, s = cases[1]
    check_close(ddf_host(x, cf, sf, 3, 1, s, "add"), oracle_forward(x, cf, sf, 3, 1, s, "add"), dtype, "ddf_host")

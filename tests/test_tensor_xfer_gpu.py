"""K1 tensor transfer kernels against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _flag(dev):
    return torch.zeros(4, dtype=torch.int64, device=dev)


@pytest.mark.parametrize("nbytes", [16, 4096, 4096 + 48, 1 << 20, (1 << 26) + 16])
def test_dense_copy_and_flag(cuda_device, nbytes):
    from execution_ucx_b200.ops import tensor_xfer as tx
    src = torch.randn(nbytes // 2, device=cuda_device).to(torch.bfloat16)
    dst = torch.zeros_like(src)
    flag = _flag(cuda_device)
    tx.push(src, dst, flag_ptr=flag.data_ptr(), flag_value=7)
    torch.cuda.synchronize()
    assert torch.equal(src.view(torch.int16), dst.view(torch.int16))
    assert int(flag[0]) == 7


@pytest.mark.parametrize("sd,dd", [(torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16),
                                   (torch.float32, torch.float8_e4m3fn), (torch.float16, torch.bfloat16),
                                   (torch.float8_e4m3fn, torch.float32)])
@pytest.mark.parametrize("n", [8, 1000, 1 << 20])
def test_cast(cuda_device, sd, dd, n):
    from execution_ucx_b200.ops import tensor_xfer as tx
    src = (torch.randn(n, device=cuda_device) * 3).to(sd)
    dst = torch.zeros(n, dtype=dd, device=cuda_device)
    tx.push(src, dst)
    torch.cuda.synchronize()
    ref = src.float().to(dd)
    assert torch.equal(dst.float(), ref.float())


@pytest.mark.parametrize("op,arg", [(1, 1.0), (2, 0.5)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_handler_epilogue(cuda_device, op, arg, dt):
    from execution_ucx_b200.ops import tensor_xfer as tx
    src = torch.rand(4099, device=cuda_device).mul(2).sub(1).to(dt)
    dst = torch.zeros_like(src)
    tx.push(src, dst, op=op, op_arg=arg)
    torch.cuda.synchronize()
    ref = (src.float() + arg if op == 1 else src.float() * arg).to(dt)
    assert torch.equal(dst.float(), ref.float())


def test_strided_gather(cuda_device):
    from execution_ucx_b200.ops import tensor_xfer as tx
    base = torch.randn(37, 64, 5, device=cuda_device)
    for view in (base.transpose(0, 2), base[:, ::3, 1:4], base.permute(1, 2, 0)[3:40:2]):
        assert not view.is_contiguous()
        dst = torch.zeros(view.numel(), dtype=torch.bfloat16, device=cuda_device)
        tx.push(view, dst)
        torch.cuda.synchronize()
        assert torch.equal(dst.float(), view.contiguous().view(-1).to(torch.bfloat16).float())
        raw = torch.zeros(view.numel(), dtype=torch.float32, device=cuda_device)
        tx.push(view, raw)
        torch.cuda.synchronize()
        assert torch.equal(raw, view.contiguous().view(-1))


def test_batch(cuda_device):
    from execution_ucx_b200.ops import tensor_xfer as tx
    g = torch.Generator(device="cpu").manual_seed(3)
    srcs, dsts, descs = [], [], []
    flags = torch.zeros(64, dtype=torch.int64, device=cuda_device)
    for i in range(40):
        n = int(torch.randint(64, 16384, (1,), generator=g))
        s = torch.rand(n, device=cuda_device) * 2 - 1
        d = torch.zeros_like(s)
        srcs.append(s), dsts.append(d)
        descs.append(tx.make_desc(s, d.data_ptr(), torch.float32, op=tx.OP_ADD, op_arg=1.0,
                                  flag_ptr=flags.data_ptr() + 8 * i, flag_value=i + 1))
    tx.push_batch(descs)
    torch.cuda.synchronize()
    for i, (s, d) in enumerate(zip(srcs, dsts)):
        assert torch.equal(d, s + 1.0)
        assert int(flags[i]) == i + 1


def test_batch_large_raw_copies(cuda_device):
    """Each descriptor of a batch is copied whole by its own CTA, also when it spans many copy blocks."""
    from execution_ucx_b200.ops import tensor_xfer as tx
    srcs, dsts, descs = [], [], []
    for i, n in enumerate((1 << 18, (1 << 20) + 40, 3 * (1 << 16) + 8, 1000)):
        s = torch.randint(0, 255, (n,), dtype=torch.uint8, device=cuda_device)
        d = torch.zeros_like(s)
        srcs.append(s), dsts.append(d)
        descs.append(tx.make_desc(s, d.data_ptr(), torch.uint8))
    tx.push_batch(descs)
    torch.cuda.synchronize()
    for s, d in zip(srcs, dsts):
        assert torch.equal(d, s)


def test_pull_batch_items_in_launch_parameters(cuda_device):
    """The transport's batched pull: every item is copied whole (aligned or not, empty, a few bytes, many
    blocks) and publishes its own flag value; more than the maximum per launch is refused."""
    from execution_ucx_b200.ops import _native, tensor_xfer as tx
    sizes = [0, 1, 15, 16, 17, 4096, 65536, 65536 + 3, 262144, 100_000] + [512 * (i + 1) for i in range(30)]
    assert len(sizes) <= _native.PULL_BATCH_MAX
    flags = torch.zeros(len(sizes), dtype=torch.int64, device=cuda_device)
    srcs, dsts, items = [], [], []
    for i, n in enumerate(sizes):
        off_s, off_d = (i % 3) * 5, (i % 4) * 3          # some of the buffers are not 16-byte aligned
        s = torch.randint(0, 255, (n + 64,), dtype=torch.uint8, device=cuda_device)
        d = torch.full((n + 64,), 7, dtype=torch.uint8, device=cuda_device)
        srcs.append(s[off_s: off_s + n]), dsts.append((d, off_d, n))
        items.append((s.data_ptr() + off_s, d.data_ptr() + off_d, n, flags.data_ptr() + 8 * i, 1000 + i))
    for rnd in range(2):
        tx.pull_batch(items)
        torch.cuda.synchronize()
        for i, (s, (d, off, n)) in enumerate(zip(srcs, dsts)):
            assert torch.equal(d[off: off + n], s)
            assert bool((d[:off] == 7).all()) and bool((d[off + n:] == 7).all())   # nothing written outside
            assert int(flags[i]) == 1000 + i
        flags.zero_()
    with pytest.raises(RuntimeError):
        tx.pull_batch(items + items)


@pytest.mark.parametrize("n", [1024, 1 << 22])   # one CTA; a grid of many CTAs, each with its own bounded wait
def test_bounded_wait_reports_timeout(cuda_device, n):
    """A wait that nothing satisfies ends by itself with a status, not a hang, and the completion
    flag is not published, however many CTAs shared the transfer."""
    from execution_ucx_b200.ops import tensor_xfer as tx
    src = torch.ones(n, device=cuda_device)
    dst = torch.zeros_like(src)
    never = _flag(cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out_flag = _flag(cuda_device)
    tx.push(src, dst, wait_flag_ptr=never.data_ptr(), wait_value=1, wait_timeout_ns=20_000_000,
            status_ptr=status.data_ptr(), flag_ptr=out_flag.data_ptr(), flag_value=5)
    torch.cuda.synchronize()
    assert int(status[0]) & 0xff == 1
    assert int(out_flag[0]) == 0 and float(dst.sum()) == 0.0
    # the context is still usable and a satisfied wait goes through
    never[0] = 1
    status.zero_()
    tx.push(src, dst, wait_flag_ptr=never.data_ptr(), wait_value=1, wait_timeout_ns=20_000_000,
            status_ptr=status.data_ptr(), flag_ptr=out_flag.data_ptr(), flag_value=5)
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and int(out_flag[0]) == 5 and torch.equal(src, dst)


def test_pingpong_loopback(cuda_device):
    from execution_ucx_b200.ops import tensor_xfer as tx
    n = 1 << 22
    a = torch.randint(0, 255, (n,), dtype=torch.uint8, device=cuda_device)
    keep = a.clone()
    b = torch.zeros_like(a)
    bar = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    ts = torch.zeros(6, dtype=torch.int64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    tx.pingpong(a, b.data_ptr(), n, 0, 0, bar, iters=5, initiator=2, ts_out=ts, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert torch.equal(a, keep) and torch.equal(b, keep)
    assert int(bar.sum()) == 0
    d = (ts[1:] - ts[:-1]).tolist()
    assert all(x > 0 for x in d)


@pytest.mark.parametrize("n,op,arg", [(2048, 0, 0.0), (1 << 20, 0, 0.0), ((1 << 22) + 24, 1, 1.5)])
def test_rpc_echo_step_single_launch(cuda_device, n, op, arg):
    """The three roles of an echo step as the phases of one launch, looped back on one GPU: the request lands in
    the request slot, the handler's result in the response slot, both flags carry the sequence number."""
    from execution_ucx_b200.ops import tensor_xfer as tx
    src = torch.randn(n, device=cuda_device).to(torch.bfloat16)
    req_slot = torch.zeros(n, dtype=torch.bfloat16, device=cuda_device)
    resp_slot = torch.zeros(n, dtype=torch.bfloat16, device=cuda_device)
    flags = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    for seq in (1, 2):
        tx.rpc_echo_step(src, req_slot.data_ptr(), flags.data_ptr(), req_slot, resp_slot.data_ptr(), flags.data_ptr() + 8,
                         flags.data_ptr(), flags.data_ptr() + 8, seq, op=[tx.OP_NONE, tx.OP_ADD][op], op_arg=arg,
                         status_ptr=status.data_ptr())
        torch.cuda.synchronize()
        assert int(status[0]) == 0 and flags.tolist() == [seq, seq]
        assert torch.equal(req_slot, src)
        want = src if op == 0 else (src.float() + arg).to(torch.bfloat16)
        assert torch.equal(resp_slot, want)
        resp_slot.zero_()
    # a request that never arrives ends the step with a status; nothing is published
    flags.zero_()
    tx.rpc_echo_step(src, req_slot.data_ptr(), flags.data_ptr() + 8, req_slot, resp_slot.data_ptr(), flags.data_ptr() + 8,
                     flags.data_ptr(), flags.data_ptr() + 8, 7, status_ptr=status.data_ptr(), wait_timeout_ns=20_000_000)
    torch.cuda.synchronize()
    assert int(status[0]) & 0xff == 1 and int(flags[0]) == 0

"""K3 MoE dispatch/combine: logical ranks emulated on one GPU, fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _routing(t, topk, n_experts, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    scores = torch.rand(t, n_experts, generator=g)
    idx = scores.topk(topk, dim=-1).indices.to(torch.int32)
    w = torch.softmax(torch.randn(t, topk, generator=g), dim=-1)
    return idx.to(dev), w.to(dev)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("world,t,hidden,topk,ne", [
    (1, 64, 512, 4, 8), (4, 96, 1024, 4, 16), (8, 40, 7168, 8, 256),
    # the general kernels: more than eight experts per token, rows wider than the streaming kernels take
    (2, 48, 1024, 12, 16), (2, 33, 9216, 4, 8), (1, 70, 1152, 8, 8)])
def test_dispatch_combine(cuda_device, fp8, world, t, hidden, topk, ne):
    """Dispatch, identity expert and gate-weighted combine against fp32 PyTorch. The streaming combine
    kernels (top-k <= 8; fp8 also hidden <= 8192) and the general ones are both reached; 1152 makes the
    last unit of a row a partial one, and odd token counts leave warps with runs of different lengths."""
    from execution_ucx_b200.ops import moe
    ranks = moe.MoeAllToAll.emulated(world, t, hidden, topk, ne, fp8=fp8)
    xs, idxs, ws = [], [], []
    for r in range(world):
        xs.append(torch.randn(t, hidden, device=cuda_device).to(torch.bfloat16))
        i, w = _routing(t, topk, ne, cuda_device, 100 + r)
        idxs.append(i), ws.append(w)
    for rnd in range(2):  # two rounds: flags and scratch must be reusable
        for r in range(world):
            ranks[r].dispatch(xs[r], idxs[r], ws[r])
        for r in range(world):
            ranks[r].expert_ready()
        outs = [ranks[r].combine().clone() for r in range(world)]
        torch.cuda.synchronize()
        for r in range(world):
            ranks[r].check_status()
            ref = moe.reference_dispatch_combine(xs[r], idxs[r], ws[r], fp8)
            torch.testing.assert_close(outs[r].float(), ref, rtol=2e-2, atol=2e-2)
        # what arrived: counts, headers and payload rows
        epr = ne // world
        for dst in range(world):
            counts = ranks[dst].recv_counts().tolist()
            for src in range(world):
                want = int(((idxs[src] // epr) == dst).sum())
                assert counts[src] == want
                if want == 0:
                    continue
                meta = ranks[dst].recv_meta(src, want).cpu()
                rows = ranks[dst].recv_rows(src, want)
                tok, kslot = meta[:, 0].long(), (meta[:, 1] & 0xffff).long()
                le = (meta[:, 1] >> 16).long()
                assert torch.equal(idxs[src].cpu()[tok, kslot].long(), le + dst * epr)
                assert bool((le[1:] >= le[:-1]).all()), "rows must be grouped by local expert"
                assert torch.equal(meta[:, 3], torch.full_like(meta[:, 3], src))
                if not fp8:
                    got = rows.view(torch.bfloat16).view(want, hidden)
                    assert torch.equal(got.view(torch.int16), xs[src][tok.to(cuda_device)].view(torch.int16))
        assert int(ranks[0].counters.sum()) >= 0


def test_capacity_overflow_is_reported(cuda_device):
    from execution_ucx_b200.ops import moe
    t, hidden, topk, ne = 32, 256, 2, 4
    (rk,) = moe.MoeAllToAll.emulated(1, t, hidden, topk, ne, capacity=16)
    x = torch.randn(t, hidden, device=cuda_device).to(torch.bfloat16)
    idx, w = _routing(t, topk, ne, cuda_device, 1)
    rk.dispatch(x, idx, w)
    torch.cuda.synchronize()
    assert int(rk.status.item()) & 0xff == 3


@pytest.mark.parametrize("world,t,hidden,topk,ne", [(4, 96, 1024, 4, 16), (8, 40, 7168, 8, 256), (2, 48, 1024, 12, 16)])
def test_combine_pairs_each_row_with_its_own_weight_and_expert(cuda_device, world, t, hidden, topk, ne):
    """A non-identity expert: every expert rank multiplies the rows it received for local expert e by
    (1 + (e + rank * experts_per_rank) / 256) before the sources combine. The fp32 reference applies the
    same factor per (token, k-slot). With the identity expert the combine is x * sum(w), and a combine that
    took another k-slot's weight, or another expert's copy of the token, would still pass; here it cannot."""
    from execution_ucx_b200.ops import moe
    ranks = moe.MoeAllToAll.emulated(world, t, hidden, topk, ne, fp8=False)
    epr = ne // world
    xs, idxs, ws = [], [], []
    for r in range(world):
        xs.append(torch.randn(t, hidden, device=cuda_device).to(torch.bfloat16))
        i, w = _routing(t, topk, ne, cuda_device, 300 + r)
        idxs.append(i), ws.append(w)
    for r in range(world):
        ranks[r].dispatch(xs[r], idxs[r], ws[r])
    for r in range(world):
        ranks[r].expert_ready()
    torch.cuda.synchronize()
    # the "expert": scale every received row in place, by its expert's factor (read from the row headers)
    for dst in range(world):
        counts = ranks[dst].recv_counts().tolist()
        for src in range(world):
            n = counts[src]
            if n == 0:
                continue
            meta = ranks[dst].recv_meta(src, n)
            le = (meta[:, 1] >> 16).long()
            factor = 1.0 + (le + dst * epr).float() / 256.0
            rows = ranks[dst].recv_rows(src, n).view(torch.bfloat16).view(n, hidden)
            rows.copy_((rows.float() * factor.unsqueeze(1)).to(torch.bfloat16))
    outs = [ranks[r].combine().clone() for r in range(world)]
    torch.cuda.synchronize()
    for r in range(world):
        ranks[r].check_status()
        x = xs[r].float()
        ref = torch.zeros_like(x)
        for k in range(topk):
            f = 1.0 + idxs[r][:, k].float() / 256.0
            y = (x * f.unsqueeze(1)).to(torch.bfloat16).float()      # what the expert stored for this (token, k)
            ref += ws[r][:, k].unsqueeze(1) * y
        torch.testing.assert_close(outs[r].float(), ref, rtol=2e-2, atol=2e-2)

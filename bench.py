#!/usr/bin/env python
"""Headline benchmark: Axon tensor-RPC bandwidth (1 GiB bf16 echo) plus the
other named workloads (latency sweep, remote-GEMM RPC, MoE dispatch+combine).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

One step = one echo RPC of a 1 GiB bf16 tensor through `AxonRuntime.invoke` on
every rank (rank r calls rank r^1's runtime; a single rank runs a server and a
client runtime on its own GPU). The timed region is bracketed by barrier +
synchronize, timed with CUDA events on the calling stream, max over ranks.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def reference_arm(args) -> int:
    # The reference is a Bazel project (no setup.py / pyproject.toml) whose build fetches OpenUCX,
    # libunifex, cista, nanobind, ... from the network; the one permitted offline install fails.
    why = ("pip install --no-index --target baseline/_ref <reference tree>: 'not installable: neither setup.py nor "
           "pyproject.toml found'; the reference builds only with Bazel plus network fetches of OpenUCX/libunifex/"
           "cista/nanobind, none of which are available offline")
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bytes", type=int, default=1 << 30, help="tensor size of the headline step")
    ap.add_argument("--no-extras", action="store_true", help="skip the sweep / GEMM / MoE side measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the data plane has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from execution_ucx_b200.models.workloads import AxonTensorRpc, TensorRpcEcho
    from execution_ucx_b200.ops import moe as moe_ops, remote_gemm as gemm_ops, tensor_xfer as tx
    from execution_ucx_b200.parallel.peer import PeerGroup
    from execution_ucx_b200.utils import timing

    group = PeerGroup.from_env() if world > 1 else PeerGroup(0, 1, dev)
    group.device = dev
    peaks = timing.measured_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    nbytes = args.bytes

    def launches() -> int:
        return tx.launch_count() + moe_ops.launch_count() + gemm_ops.launch_count()

    def sync_all():
        torch.cuda.synchronize()
        group.barrier()
        torch.cuda.synchronize()

    import asyncio

    src = torch.randn(nbytes // 2, device=dev).to(torch.bfloat16)       # N(0,1) bf16, larger than L2
    host_in = torch.empty(nbytes // 2, dtype=torch.bfloat16).pin_memory()
    host_in.copy_(src.cpu())
    host_out = torch.empty(nbytes // 2, dtype=torch.bfloat16).pin_memory()
    dev_in = torch.empty_like(src)
    res = {}

    # ---------------- headline: the echo RPC through the public API ----------------
    # One step = `await AxonRuntime.invoke(tensor, function="echo")` on every rank at once, each to its
    # partner's runtime (a Python handler registered with `register_function`), device tensors both ways.
    # The bytes move by the runtime's transfer kernels (pushed by the sender's kernel into the buffer the
    # receiver's memory policy returned; completion through a flag the receiver's worker thread polls).
    async def api_main():
        api = AxonTensorRpc(group)
        await api.start(connect_all=not args.no_extras)
        for _ in range(warmup):
            y = await api.step(src)
        torch.cuda.synchronize()
        await api.barrier()
        if sampler:
            sampler.mark()
        l0 = api.kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            y = await api.step(src)       # resolves when the reply has landed in this rank's buffer
        e1.record()
        torch.cuda.synchronize()
        res["host_ms"] = (time.perf_counter() - t0) * 1e3
        res["event_ms"] = e0.elapsed_time(e1)
        res["launches"] = api.kernel_launches() - l0
        await api.barrier()
        res["echo_ok"] = bool(torch.equal(y.view(torch.int16), src.view(torch.int16)))      # every byte of the last reply
        res["stats"] = api.transport_stats()

        # ---- end to end: pinned host -> device, the RPC, the whole reply device -> pinned host, every step ----
        async def e2e_step():
            dev_in.copy_(host_in, non_blocking=True)
            r = await api.step(dev_in)
            host_out.copy_(r, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(host_out[0])

        e2e_steps = max(3, min(steps, 10))
        for _ in range(3):
            await e2e_step()
        torch.cuda.synchronize()
        await api.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            await e2e_step()
        torch.cuda.synchronize()
        res["e2e_ms"] = (time.perf_counter() - t0) * 1e3 / e2e_steps
        await api.barrier()
        res["e2e_ok"] = bool(torch.equal(host_out.view(torch.int16), host_in.view(torch.int16)))
        # ---- the same call at every size (no host copies): latency and bandwidth of the RPC layer ----
        rows = []
        if not args.no_extras:
            for lg in range(12, 31):
                n = min(1 << lg, nbytes)
                x = src[: n // 2]
                iters = 100 if lg <= 20 else (20 if lg <= 26 else 5)
                for _ in range(3):
                    await api.step(x)
                await api.barrier()
                ts = []
                for _ in range(iters):
                    t = time.perf_counter()
                    y = await api.step(x)
                    ts.append((time.perf_counter() - t) * 1e6)
                del y
                await api.barrier()
                ts.sort()
                p50 = group.max_over_ranks(ts[len(ts) // 2])
                p99 = group.max_over_ranks(ts[min(len(ts) - 1, int(len(ts) * 0.99))])
                rows.append({"bytes": n, "rtt_p50_us": round(p50, 1), "rtt_p99_us": round(p99, 1),
                             "one_way_GBps": round(n / (p50 / 2 * 1e-6) / 1e9, 2)})
                if n == nbytes:
                    break
        res["api_rows"] = rows
        if not args.no_extras:
            try:
                res["services"] = await service_measurements(api, group, peaks)
            except Exception as e:  # a failed side measurement must not hide the headline
                traceback.print_exc()
                res["services"] = {"error": f"{type(e).__name__}: {e}", "trace": traceback.format_exc(limit=4)}
        api.stop()

    # the sampler starts (and loads NVML) before the barrier, so that no rank enters the timed region late
    sampler = timing.ClockSampler(local_rank).start() if rank == 0 else None
    asyncio.run(api_main())
    clocks = sampler.stop() if sampler else None
    gpu_launches = res["launches"]
    # CUDA events on the calling stream bracket the steps (the kernels themselves run on the runtimes' streams,
    # in this process and in the partner's); the host clock around the same region is reported beside them
    ms_total = group.max_over_ranks(res["event_ms"])
    ms_per_step = ms_total / steps
    one_way_gbs_per_rank = nbytes / (ms_per_step / 2 * 1e-3) / 1e9
    value = one_way_gbs_per_rank * world
    echo_ok = bool(group.max_over_ranks(0.0 if res["echo_ok"] else 1.0) == 0.0)
    e2e_ms = group.max_over_ranks(res["e2e_ms"])
    e2e = {"value": round(nbytes / (e2e_ms / 2 * 1e-3) / 1e9 * world, 2), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": host_in.numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2,
           "api": "execution_ucx_b200.axon.AxonRuntime.invoke('echo'): request copied from pinned host memory, whole reply copied back",
           "echo_verified": bool(group.max_over_ranks(0.0 if res["e2e_ok"] else 1.0) == 0.0),
           "timing": "host clock around the steps, max over ranks"}
    del host_in, host_out, dev_in

    extra = {"api_sweep": {"what": "AxonRuntime.invoke('echo') of a device tensor, every rank to its partner at once; host clock per call, max over ranks",
                           "rows": res["api_rows"]},
             "headline_host_clock_ms_per_step": round(group.max_over_ranks(res["host_ms"]) / steps, 5),
             "transport_counters_rank0": res["stats"], **res.get("services", {})}
    if not args.no_extras:
        # the data plane alone (no header, no dispatcher, no runtime): what the kernels do when nothing else is in the way
        rpc = TensorRpcEcho(group, nbytes)
        extra.update(side_measurements(group, dev, rank, world, peaks, rpc, src))
        rpc.close()
        del rpc
    del src

    if rank == 0:
        out = {
            "metric": "axon_tensor_rpc_unidirectional_GBps", "value": round(value, 2), "unit": "GB/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic N(0,1) bf16, random-init weights",
            "config": {"model": "axon tensor-RPC echo ping-pong (BASELINE config 2)", "message_bytes": nbytes,
                       "global_batch": world, "seq_len": nbytes // 2, "parallelism": f"p2p-pairs{world}",
                       "path": "AxonRuntime.invoke -> RPC header -> active message -> transfer kernel -> Python handler -> and back",
                       "pairing": "rank r <-> r^1; n_gpus=1 is two runtimes on one GPU (a loopback through the same code)",
                       "scaling_note": "n_gpus=1 moves the bytes inside one GPU's HBM, n_gpus>=2 across NVLink (770 GB/s "
                                       "measured per direction and GPU): the 1-GPU value is not the base of the multi-GPU ones",
                       "l2": "inputs (1 GiB) larger than L2; no flush needed"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": gpu_launches, "echo_verified": echo_ok,
            "peaks": {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained", "source")},
            "extra": extra,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


async def service_measurements(api, group, peaks):
    """Remote-GEMM RPC and MoE dispatch+combine through the runtime: the GEMM is an Axon function of the
    callee (`AxonRuntime.serve_gemm` / `remote_gemm`), the MoE buffers were announced by Axon calls."""
    import torch
    from execution_ucx_b200.models.workloads import MoeAxon, RemoteGemmAxon
    from execution_ucx_b200.utils import timing
    world = group.world
    out = {}
    m = n = k = 8192
    flush = timing.L2Flusher(group.device)

    async def timed_calls(w, iters=10, warm=3):
        ts = []
        for i in range(warm + iters):
            flush()
            torch.cuda.synchronize()
            await api.barrier()
            t0 = time.perf_counter()
            await w.step()
            if i >= warm:
                ts.append((time.perf_counter() - t0) * 1e3)
        return group.max_over_ranks(timing.percentile(ts, 50))

    wid = 20
    for fmt, key in (("bf16", "remote_gemm_axon_bf16"), ("fp8_block", "remote_gemm_axon_fp8_block_scaled"),
                     ("fp8_block_pow2", "remote_gemm_axon_fp8_block_scaled_pow2"), ("mxfp8", "remote_gemm_axon_mxfp8")):
        wid += 1
        w = RemoteGemmAxon(api, m, n, k, fmt=fmt, weight_id=wid)
        await api.barrier()
        ms = await timed_calls(w)
        err = group.max_over_ranks(w.max_abs_err(256))
        t_compute = 2.0 * m * n * k / (peaks["bf16_tflops"] * 1e12) * 1e3
        x_bytes = m * k * (2 if fmt == "bf16" else 1)
        t_link = x_bytes / (timing.NVLINK_PEER_GBS * 1e9) * 1e3 if world > 1 else 0.0
        out[key] = {"shape": [m, n, k], "ms_p50": round(ms, 4), "tflops_per_gpu": round(2.0 * m * n * k / (ms * 1e-3) / 1e12, 1),
                    "roofline_ms_vs_bf16_peak": round(max(t_compute, t_link), 4),
                    "fraction_of_bf16_roofline_of_" + peaks.get("source", "measured"): round(max(t_compute, t_link) / ms, 3),
                    "max_abs_err_vs_fp32_first_256_rows": err,
                    "timing": "host clock around `await remote_gemm(...)` (request, kernel, reply), max over ranks",
                    "path": "Axon call with the caller's region descriptors -> callee's handler launches the GEMM on the caller's memory -> reply"}
        if fmt == "fp8_block_pow2":
            out[key]["format"] = ("e4m3 + fp32 scale per 1x128 (X) and 128x128 (W), every scale a power of two: routed to the MX kernel, "
                                  "where the tensor core applies the scales; same product as fp8_block_scaled")
        del w
    if world > 2:
        w = RemoteGemmAxon(api, m, n, k, fmt="bf16", peers="all", weight_id=30)
        await api.barrier()
        ms = await timed_calls(w, iters=5, warm=2)
        calls = world - 1
        out["remote_gemm_axon_bf16_all_peers"] = {"shape": [m, n, k], "calls_served_per_rank": calls, "ms_per_round_p50": round(ms, 3),
                                                   "ms_per_call": round(ms / calls, 4), "max_abs_err_vs_fp32_first_256_rows": group.max_over_ranks(w.max_abs_err(256)),
                                                   "tflops_per_gpu": round(2.0 * m * n * k * calls / (ms * 1e-3) / 1e12, 1)}
        del w
    torch.cuda.empty_cache()
    for fp8, key in ((False, "moe_axon_bf16"), (True, "moe_axon_fp8")):
        mo = await MoeAxon.create(api, fp8=fp8)
        ts = timing.time_cuda(mo.step, iters=10, warmup=3, flush=flush, before=group.barrier if world > 1 else None)
        mo.a2a.check_status()
        us = group.max_over_ranks(timing.percentile(ts, 50)) * 1e3
        err = float((mo.a2a.out.float() - mo.reference()).abs().max())
        remote = mo.bytes_per_direction() * (world - 1) / world
        if world > 1:
            roof_us = 2 * remote / (timing.NVLINK_PEER_GBS * 1e9) * 1e6
            bound = "nvlink (measured 770 GB/s per direction)"
        else:
            roof_us = 2 * (mo.bytes_per_direction() + mo.x.numel() * 2) / (peaks["hbm_gbs"] * 1e9) * 1e6
            bound = "hbm copy (read+write)"
        out[key] = {"dispatch_combine_us_p50": round(us, 1), "roofline_us": round(roof_us, 1), "bound": bound,
                    "fraction_of_roofline": round(roof_us / us, 3), "max_abs_err": err, "tokens_per_rank": mo.a2a.n_tokens,
                    "hidden": mo.a2a.hidden, "topk": mo.a2a.topk, "experts": mo.a2a.n_experts,
                    "buffers": "allocated from the runtime's CUDA memory resource, announced to the peers by Axon calls"}
        await mo.close()
    return out


def side_measurements(group, dev, rank, world, peaks, rpc, src):
    """Latency sweep, remote-GEMM RPC and MoE dispatch+combine (each device-timed, max over ranks)."""
    import torch
    from execution_ucx_b200.models.workloads import DevicePingPong, MoeDispatchCombine, RemoteGemmRpc
    from execution_ucx_b200.utils import timing
    extra = {}
    flush = timing.L2Flusher(dev)

    def guarded(name, fn):
        try:
            extra[name] = fn()
        except Exception as e:  # a failed side measurement must not hide the headline
            extra[name] = {"error": f"{type(e).__name__}: {e}", "trace": traceback.format_exc(limit=3)}
        torch.cuda.synchronize()
        group.barrier()

    def sweep():
        pp = DevicePingPong(group, 1 << 30)
        rows = []
        for lg in range(12, 31):
            n = 1 << lg
            iters = 200 if lg <= 20 else (50 if lg <= 26 else 10)
            pp.run(n, 5)
            group.barrier()
            rtt = pp.run(n, iters).float()
            group.barrier()
            p50 = group.max_over_ranks(float(rtt.median())) / 1e3
            p99 = group.max_over_ranks(float(rtt.quantile(0.99))) / 1e3
            rows.append({"bytes": n, "rtt_p50_us": round(p50, 2), "rtt_p99_us": round(p99, 2),
                         "one_way_GBps": round(n / (p50 / 2 * 1e-6) / 1e9, 2)})
        pp.close()
        return {"timing": "device globaltimer inside one persistent kernel per GPU", "rows": rows}

    def rpc_sweep():
        """Round trips are serialised by their data, so a sample times a run of them between two events
        and divides: the ranks' launch skew (tens of microseconds after a host barrier) would otherwise
        be most of a small message's figure. L2 is flushed between samples."""
        rows = []
        for lg in (12, 16, 20, 24, 28, 30):
            n = 1 << lg
            if n > src.numel() * 2:
                break
            s = src[: n // 2]
            inner = 32 if lg <= 20 else (8 if lg == 24 else 2)

            def run_steps():
                for _ in range(inner):
                    rpc.step(s)
            ts = timing.time_cuda(run_steps, iters=12, warmup=2, flush=flush, before=group.barrier if world > 1 else None)
            ts = [t / inner for t in ts]
            p50 = group.max_over_ranks(timing.percentile(ts, 50)) * 1e3
            p99 = group.max_over_ranks(timing.percentile(ts, 99)) * 1e3
            rows.append({"bytes": n, "steps_per_sample": inner, "rtt_p50_us": round(p50, 2), "rtt_p99_us": round(p99, 2),
                         "one_way_GBps": round(n / (p50 / 2 * 1e-6) / 1e9, 2)})
        return {"what": "the data plane alone: no header, no dispatcher, no runtime; buffers exchanged once at set-up",
                "timing": "CUDA events around a run of steps, one launch per step and rank (request push, handler + push "
                          "back, completion wait as phases of one kernel), divided by the number of steps", "rows": rows}

    def gemm(fp8):
        def run():
            m = n = k = 8192
            w = RemoteGemmRpc(group, m, n, k, fp8=fp8)
            ts = timing.time_cuda(w.step, iters=10, warmup=3, flush=flush, before=group.barrier if world > 1 else None)
            w.check()
            ms = group.max_over_ranks(timing.percentile(ts, 50))
            tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            # denominator: the measured cuBLAS bf16 burst; fp8 is reported against the same figure (no measured fp8 peak)
            t_compute = 2.0 * m * n * k / (peaks["bf16_tflops"] * 1e12) * 1e3
            x_bytes = m * k * (1 if fp8 else 2) + (m * (k // 128) * 4 if fp8 else 0)  # MX scales: m * k / 32, the same count
            t_link = x_bytes / (timing.NVLINK_PEER_GBS * 1e9) * 1e3 if world > 1 else 0.0
            err = float((w.y[:256].float() - w.reference_rows(256)).abs().max()) if world == 1 else None
            w.close()
            out8 = {}
            if fp8:
                # there is no measured fp8 GEMM peak to go by: the nominal dense figure, labelled as such
                t8 = max(2.0 * m * n * k / 4.5e15 * 1e3, t_link)
                out8 = {"roofline_ms_vs_nominal_fp8_peak_4500": round(t8, 4), "fraction_of_nominal_fp8_roofline": round(t8 / ms, 3),
                        "format": "MXFP8: e4m3 + UE8M0 scale per 32 elements, scaled in the tensor core" if fp8 == "mx"
                        else "e4m3 + fp32 scale per 1x128 (X) and 128x128 (W), applied in the epilogue"}
            return {"shape": [m, n, k], "ms_p50": round(ms, 4), "tflops_per_gpu": round(tf, 1), **out8,
                    "roofline_ms_vs_bf16_peak": round(max(t_compute, t_link), 4),
                    "fraction_of_bf16_roofline_of_" + peaks.get("source", "measured"): round(max(t_compute, t_link) / ms, 3),
                    "max_abs_err_vs_fp32_first_256_rows": err,
                    "x_source": "partner GPU's memory, pulled panel by panel inside the GEMM kernel" if world > 1
                    else "same GPU, read in place"}
        return run

    def gemm_all_peers():
        """Every rank is caller of every other rank's GEMM and callee for every other rank."""
        from execution_ucx_b200.models.workloads import RemoteGemmAllPeers
        if world < 3:
            return {"skipped": "same as the pair measurement below three ranks"}
        m = n = k = 8192
        w = RemoteGemmAllPeers(group, m, n, k)
        ts = timing.time_cuda(w.step, iters=5, warmup=2, flush=flush, before=group.barrier)
        w.check()
        ms = group.max_over_ranks(timing.percentile(ts, 50))
        calls = world - 1
        w.close()
        return {"shape": [m, n, k], "calls_served_per_rank": calls, "ms_per_round_p50": round(ms, 3),
                "ms_per_call": round(ms / calls, 4), "tflops_per_gpu": round(2.0 * m * n * k * calls / (ms * 1e-3) / 1e12, 1)}

    def moe(fp8):
        def run():
            w = MoeDispatchCombine(group, fp8=fp8)
            ts = timing.time_cuda(w.step, iters=10, warmup=3, flush=flush, before=group.barrier if world > 1 else None)
            w.a2a.check_status()
            us = group.max_over_ranks(timing.percentile(ts, 50)) * 1e3
            err = float((w.a2a.out.float() - w.reference()).abs().max())
            remote = w.bytes_per_direction() * (world - 1) / world
            x_numel, dirbytes = w.x.numel(), w.bytes_per_direction()
            w.a2a.close()
            if world > 1:
                roof_us = 2 * remote / (timing.NVLINK_PEER_GBS * 1e9) * 1e6
                bound = "nvlink (measured 770 GB/s per direction)"
            else:
                x_bytes = x_numel * 2
                roof_us = 2 * (dirbytes + x_bytes) / (peaks["hbm_gbs"] * 1e9) * 1e6
                bound = "hbm copy (read+write)"
            return {"dispatch_combine_us_p50": round(us, 1), "roofline_us": round(roof_us, 1), "bound": bound,
                    "fraction_of_roofline": round(roof_us / us, 3), "max_abs_err": err,
                    "tokens_per_rank": w.a2a.n_tokens, "hidden": w.a2a.hidden, "topk": w.a2a.topk,
                    "experts": w.a2a.n_experts}
        return run

    def baselines():
        """The same three workloads with library calls only (NCCL, cuBLAS through torch)."""
        from execution_ucx_b200.models import baselines as bl
        out = {"note": "library baselines measured in this run: none of this package's kernels on these paths"}
        n = src.numel() * 2
        echo = bl.NcclEcho(rank, world, n, dev)
        ts = timing.time_cuda(lambda: echo.step(src), iters=10, warmup=3, before=group.barrier if world > 1 else None)
        ms = group.max_over_ranks(timing.percentile(ts, 50))
        out["echo_1GiB"] = {"what": "NCCL send/recv there and back" if world > 1 else "two torch D2D copies",
                            "ms_p50": round(ms, 4), "one_way_GBps_aggregate": round(n / (ms / 2 * 1e-3) / 1e9 * world, 1)}
        del echo
        m = nn = k = 8192
        gm = bl.RecvGemmSend(rank, world, m, nn, k, dev)
        ts = timing.time_cuda(gm.step, iters=10, warmup=3, flush=flush, before=group.barrier if world > 1 else None)
        ms = group.max_over_ranks(timing.percentile(ts, 50))
        out["remote_gemm_bf16"] = {"what": "NCCL recv X + cuBLAS + NCCL send Y" if world > 1 else "cuBLAS (torch.matmul)",
                                   "ms_p50": round(ms, 4), "tflops_per_gpu": round(2.0 * m * nn * k / (ms * 1e-3) / 1e12, 1)}
        del gm
        try:
            sm = bl.ScaledMmBaseline(m, nn, k, dev)
            ts = timing.time_cuda(sm.step, iters=10, warmup=3, flush=flush)
            ms = group.max_over_ranks(timing.percentile(ts, 50))
            out["gemm_fp8_scaled_mm"] = {"what": "torch._scaled_mm (cuBLASLt), e4m3 x e4m3, per-tensor scales, local operands",
                                         "ms_p50": round(ms, 4), "tflops_per_gpu": round(2.0 * m * nn * k / (ms * 1e-3) / 1e12, 1)}
            del sm
        except Exception as e:
            out["gemm_fp8_scaled_mm"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        # ping-pong at every size: NCCL send/recv there and back, and the copy engine (cudaMemcpyPeerAsync, one way, doubled)
        pp = bl.PingPongSweep(group, src.numel() * 2)
        rows = []
        for lg in range(12, 31):
            nb = 1 << lg
            if nb > src.numel() * 2:
                break
            sv = src[: nb // 2]
            iters = 30 if lg <= 24 else 8
            tn = timing.time_cuda(lambda: pp.nccl_round_trip(sv), iters=iters, warmup=3, before=group.barrier if world > 1 else None)
            tc = timing.time_cuda(lambda: pp.copy_engine_one_way(sv), iters=iters, warmup=3, before=group.barrier if world > 1 else None)
            n50 = group.max_over_ranks(timing.percentile(tn, 50)) * 1e3
            n99 = group.max_over_ranks(timing.percentile(tn, 99)) * 1e3
            c50 = group.max_over_ranks(timing.percentile(tc, 50)) * 1e3 * 2
            rows.append({"bytes": nb, "nccl_rtt_p50_us": round(n50, 1), "nccl_rtt_p99_us": round(n99, 1),
                         "nccl_one_way_GBps": round(nb / (n50 / 2 * 1e-6) / 1e9, 2),
                         "copy_engine_2x_one_way_us": round(c50, 1), "copy_engine_GBps": round(nb / (c50 / 2 * 1e-6) / 1e9, 2)})
        pp.close()
        out["pingpong_sweep"] = {"timing": "CUDA events around one call, launch included, max over ranks; both ranks of a pair at once",
                                 "rows": rows}
        w = MoeDispatchCombine(group, fp8=False)
        mo = bl.AllToAllMoe(rank, world, w.x, w.idx, w.w, w.a2a.n_experts)
        ts = timing.time_cuda(mo.step, iters=10, warmup=3, flush=flush, before=group.barrier if world > 1 else None)
        us = group.max_over_ranks(timing.percentile(ts, 50)) * 1e3
        err = float((mo.out.float() - w.reference()).abs().max())
        out["moe_bf16"] = {"what": "torch sort/gather + all_to_all_single x2 + index_add_", "dispatch_combine_us_p50": round(us, 1),
                           "max_abs_err": err}
        w.a2a.close()
        return out

    def rpc_storm():
        """All-to-all small-message RPC storm through the C++ runtime: every rank serves `+1.0` on an fp32
        device tensor and keeps 64 calls in flight to every other rank (sizes log-uniform 256 B - 64 KiB)."""
        import re
        import shutil
        import subprocess
        import tempfile
        import torch.distributed as dist
        if world < 2:
            return {"skipped": "needs at least two ranks"}
        binary = ROOT / "execution_ucx_b200" / "_lib" / "eux_axon_rpc_perf"
        box = [tempfile.mkdtemp(prefix="eux_mesh_") if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        out = subprocess.run([str(binary), "--mesh", "--rank", str(rank), "--world", str(world), "--dir", box[0], "-m", "cuda",
                              "-d", str(dev.index), "-n", "4000", "-o", "64"], capture_output=True, text=True, timeout=300)
        group.barrier()
        if rank == 0:
            shutil.rmtree(box[0], ignore_errors=True)
        m = re.search(r"calls=(\d+) failed=(\d+) seconds=([\d.]+) calls_per_s=([\d.]+) payload_GBps=([\d.]+) p50_us=([\d.]+) p99_us=([\d.]+)", out.stdout)
        if not m:
            raise RuntimeError("storm failed: " + (out.stderr or out.stdout)[-500:])
        calls, failed, secs, cps, gbps, p50, p99 = (float(x) for x in m.groups())
        t = torch.tensor([cps, gbps, failed], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        return {"calls_per_s_all_ranks": round(float(t[0])), "payload_GBps_all_ranks": round(float(t[1]), 2),
                "failed": int(t[2]), "p50_us_max_over_ranks": round(group.max_over_ranks(p50), 1),
                "p99_us_max_over_ranks": round(group.max_over_ranks(p99), 1), "outstanding_per_ordered_pair": 64,
                "calls_per_rank_per_peer": 4000, "timing": "host clock inside eux_axon_rpc_perf --mesh (one process per GPU)"}

    guarded("latency_sweep_device", sweep)
    guarded("tensor_rpc_sweep", rpc_sweep)
    guarded("remote_gemm_rpc_bf16", gemm(False))
    guarded("remote_gemm_rpc_fp8_block_scaled", gemm(True))
    guarded("remote_gemm_rpc_mxfp8", gemm("mx"))
    guarded("remote_gemm_rpc_bf16_all_peers", gemm_all_peers)
    guarded("moe_bf16", moe(False))
    guarded("moe_fp8", moe(True))
    guarded("library_baselines", baselines)
    guarded("small_rpc_storm_all_to_all", rpc_storm)
    return extra


if __name__ == "__main__":
    sys.exit(main())

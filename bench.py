"""Benchmark of the binary-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload mlp_stack|gemm_sweep] [--tokens T]

Default workload (`mlp_stack`): the 7B-width converted-MLP stack -- 8 SwiGLU blocks,
d = 4096, ffn = 14336, every matrix binary, bf16 activations N(0,1), 16384 tokens
per GPU, AdamW on the row scales, QSTEOptimizer on the coordinates, coordinate
evidence all-reduced across ranks every step.  One step = forward + backward
(coordinate updates run inside backward) + both optimizer steps.  Data is
synthetic and weights are random-init.

Prints ONE JSON line.  `value` is whole-job training tokens/s with the inputs
already in HBM; `e2e` is the same step fed from pinned host memory with the loss
read back every step; `roofline` is the dominant kernel (the packed-sign forward
GEMM of the up projection) timed alone with CUDA events; `cpu_baseline` is the
reference's own CPU kernels (oracle/_ref, else the oracle port) on one block and a
bounded token sample, on this box's host cores.

`--impl reference` times that CPU path as the whole arm.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from contextlib import nullcontext
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402
import torch.nn as nn  # noqa: E402
import torch.nn.functional as F  # noqa: E402

D_MODEL, D_FFN, BLOCKS, TOKENS = 4096, 14336, 8, 16384
METRIC = "converted_mlp_train_tokens_per_s"
SWEEP_SHAPES = [(4096, 11008), (11008, 4096), (4096, 14336), (14336, 4096)]
SWEEP_BATCHES = [1, 16, 128, 4096, 16384]


def stack_config(blocks: int, tokens: int, world: int) -> dict:
    """`config` of the default workload, the same words on both arms."""

    return {
        "workload": f"converted SwiGLU MLP stack: {blocks} blocks, d={D_MODEL}, ffn={D_FFN}, "
                    f"{tokens} tokens per GPU, all {3 * blocks} matrices binary, evidence all-reduce per step",
        "tokens_per_gpu": tokens, "parallelism": f"dp{world}",
        "l2": "inputs larger than L2 (134 MB of activations per step, two rotating batches)",
    }


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"],
                "bf16_tflops_sustained": data.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------
# the workload (harness code: plain PyTorch around the converted layers)
# ------------------------------------------------------------------------------------------

class SwiGLU(nn.Module):
    def __init__(self, dim: int, ffn: int, device):
        super().__init__()
        self.gate = nn.Linear(dim, ffn, bias=False, device=device)
        self.up = nn.Linear(dim, ffn, bias=False, device=device)
        self.down = nn.Linear(ffn, dim, bias=False, device=device)
        # a module, not F.silu: convert(activations=True) swaps it for the packed SiLU, which
        # keeps an int8 derivative tape instead of the bf16 pre-activation
        self.act = nn.SiLU()

    def forward(self, x):
        h = F.rms_norm(x, (x.shape[-1],))
        return x + self.down(self.act(self.gate(h)) * self.up(h))


class Stack(nn.Module):
    def __init__(self, blocks: int, dim: int, ffn: int, device):
        super().__init__()
        self.blocks = nn.ModuleList([SwiGLU(dim, ffn, device) for _ in range(blocks)])

    def forward(self, x):
        for block in self.blocks:
            x = block(x)
        return x


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _run(self):
        nvml = self._nvml
        names = {
            "hw_slowdown": getattr(nvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "sw_power_cap": getattr(nvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_thermal_slowdown": getattr(nvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "hw_power_brake_slowdown": getattr(nvml, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nvml.nvmlDeviceGetClockInfo(self._handle, nvml.NVML_CLOCK_SM))
                mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                self.reasons.update(name for name, bit in names.items() if mask & bit)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def step_trace(step, steps: int = 2) -> dict:
    """Where a step's time goes: `steps` steps under the torch profiler (kernel times from CUPTI,
    not a benchmark number), grouped by kind of kernel, with the busy and idle time of the
    busiest stream (the compute stream).  Milliseconds per step."""

    import collections

    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as trace:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    events = [e for e in trace.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    duration = lambda e: e.device_time if hasattr(e, "device_time") else e.cuda_time  # noqa: E731
    groups, streams = collections.Counter(), collections.defaultdict(list)
    kinds = (("packed_gemm_tc", "packed-sign GEMMs"), ("prepare_rows", "gradient pre-pass"),
             ("pack_affine", "pack_affine_rows"), ("smooth_", "packed activation kernels"),
             ("split_finish", "GEMM tail kernels"), ("finish_inner", "GEMM tail kernels"),
             ("nccl", "NCCL collectives"), ("Memcpy", "copies"))
    update = ("row_squares", "column_squares", "precondition", "moment_", "coordinate_and_pack", "finish_factors",
              "finish_update_norm", "finish_moment_norm", "commit_scales", "publish_flips")
    for e in events:
        name = e.name
        kind = next((label for key, label in kinds if key in name), None)
        if kind is None:
            kind = "coordinate update kernels" if any(key in name for key in update) else \
                "torch kernels (harness element-wise, norms, loss, AdamW)"
        groups[kind] += duration(e)
        streams[getattr(e, "device_resource_id", None)].append((e.time_range.start, e.time_range.end))
    busiest = max(streams.values(), key=lambda spans: sum(b - a for a, b in spans))
    busiest.sort()
    idle = sum(max(0.0, busiest[i + 1][0] - busiest[i][1]) for i in range(len(busiest) - 1))
    begin, end = min(a for spans in streams.values() for a, _ in spans), max(b for spans in streams.values() for _, b in spans)
    per_step = lambda us: round(us / steps / 1e3, 3)  # noqa: E731
    return {"steps": steps, "span_ms": per_step(end - begin),
            "compute_stream_busy_ms": per_step(sum(b - a for a, b in busiest)), "compute_stream_idle_ms": per_step(idle),
            "compute_stream_launches": len(busiest) // steps,
            "other_streams_busy_ms": per_step(sum(b - a for spans in streams.values() if spans is not busiest for a, b in spans)),
            "kernel_ms_by_kind": {kind: per_step(us) for kind, us in groups.most_common()}}


def launch_count() -> int:
    from qste_b200.kernels import _cabi

    return int(_cabi.load().qste_b200_launch_count())


def timed(fn, steps: int, stream=None) -> float:
    """Seconds for `steps` calls of fn, by CUDA events on the current stream."""

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1e3


def max_over_ranks(seconds: float, world: int, device) -> float:
    if world == 1:
        return seconds
    import torch.distributed as dist

    value = torch.tensor([seconds], dtype=torch.float64, device=device)
    dist.all_reduce(value, op=dist.ReduceOp.MAX)
    return float(value.item())


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------

def run_ours(args) -> dict:
    import qste_b200 as qste
    from qste_b200 import distributed as qdist
    from qste_b200 import kernels

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    tokens = args.tokens or TOKENS
    blocks = args.blocks or BLOCKS

    torch.manual_seed(1234)  # same weights on every rank
    model = Stack(blocks, D_MODEL, D_FFN, device)
    qste.convert(model, include=["blocks.*.gate", "blocks.*.up", "blocks.*.down"])
    # The backward GEMMs (only those: no collective is in flight during forward) leave a few SMs
    # to the evidence all-reduce that runs beside them; without that NCCL's blocks wait for a
    # GEMM to end and the next GEMM's blocks then start late.
    reducer = qdist.mean_evidence(overlap=True, reserve_sms=args.reserve if args.reserve >= 0 else None) \
        if world > 1 else None
    coordinates = qste.QSTEOptimizer(model, gradient_reducer=reducer if reducer else False, async_update=True)
    floats = list(qste.continuous_parameters(model))
    host_optimizer = torch.optim.AdamW(floats, lr=1e-3, fused=True)

    generator = torch.Generator(device=device).manual_seed(1000 + rank)  # different data per rank
    pool = [torch.randn(tokens, D_MODEL, device=device, dtype=torch.bfloat16, generator=generator)
            for _ in range(2)]
    pinned = [x.cpu().pin_memory() for x in pool]
    # end-to-end feed: two staging buffers, the next batch copied from pinned host memory on a copy
    # stream while the current step runs (what a loader with pinned memory does)
    staging = [torch.empty_like(pool[0]) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device)
    arrived = [torch.cuda.Event() for _ in range(2)]
    released = [torch.cuda.Event() for _ in range(2)]
    for event in released:
        event.record()
    counter = {"step": 0, "flips": 0, "fed": 0}

    def reduce_float_grads():
        if world == 1:
            return
        import torch.distributed as dist

        flat = torch.cat([p.grad.reshape(-1) for p in floats])
        dist.all_reduce(flat)
        flat.div_(world)
        offset = 0
        for p in floats:
            p.grad.copy_(flat[offset:offset + p.numel()].view_as(p.grad))
            offset += p.numel()

    def step(x):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(x).float().square().mean()
        loss.backward()
        reduce_float_grads()
        host_optimizer.step()
        counter["flips"] += coordinates.step()
        host_optimizer.zero_grad(set_to_none=True)
        coordinates.zero_grad()
        counter["step"] += 1
        return loss

    def resident_step():
        step(pool[counter["step"] % len(pool)])

    def prefetch(index):
        slot = index % 2
        copy_stream.wait_event(released[slot])  # the step that read this buffer is done with it
        with torch.cuda.stream(copy_stream):
            staging[slot].copy_(pinned[index % len(pinned)], non_blocking=True)
            arrived[slot].record(copy_stream)

    def e2e_step():
        # one host-to-device copy issued and one loss read back per step; the copy that this step
        # consumes was issued by the step before, the one it issues feeds the next
        index = counter["fed"]
        slot = index % 2
        torch.cuda.current_stream(device).wait_event(arrived[slot])
        prefetch(index + 1)
        loss = step(staging[slot])
        released[slot].record()
        counter["fed"] = index + 1
        return float(loss.item())

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        resident_step()
    barrier()
    launches_before = launch_count()
    with ClockSampler(local) as clocks:
        seconds = timed(resident_step, args.steps)
    launches = launch_count() - launches_before
    barrier()
    seconds = max_over_ranks(seconds, world, device)

    prefetch(0)
    e2e_step()
    barrier()
    e2e_seconds = max_over_ranks(timed(e2e_step, args.steps), world, device)

    result = {
        "metric": METRIC, "value": world * tokens * args.steps / seconds, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * seconds / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (N(0,1) activations, random-init weights)",
        "config": stack_config(blocks, tokens, world),
        "e2e": {"value": world * tokens * args.steps / e2e_seconds, "unit": "tokens/s",
                "h2d_bytes_per_step": staging[0].numel() * staging[0].element_size(), "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "flips_per_step": counter["flips"] / max(1, counter["step"]),
        "wait_timeouts": kernels.wait_timeouts(device),
        "ranks_agree": bool(qdist.surfaces_agree(model)),
    }
    if args.trace and rank == 0 and world == 1:
        result["trace"] = step_trace(resident_step)
    if rank == 0 and not args.no_extras:
        # the kernels below are timed alone, against the burst peak: let the part leave the power
        # cap the step drove it into before timing them
        torch.cuda.synchronize()
        time.sleep(5.0)
        result["roofline"] = kernel_roofline(device, tokens)
        if world == 1:
            # the per-kernel table and the CPU baseline belong to the one-GPU line; at N > 1 the
            # other ranks would only wait for them
            result["kernels"] = kernel_breakdown(device, tokens)
            result["cpu_baseline"] = cpu_baseline(tokens)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return result if rank == 0 else {}


def _gemm_inputs(device, m, k, n, seed=2):
    generator = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(m, k, device=device, dtype=torch.bfloat16, generator=generator)
    bits = torch.randint(0, 256, (n, k // 8), device=device, dtype=torch.uint8, generator=generator)
    scale = torch.rand(n, device=device, generator=generator) * 0.04 + 0.01
    return x, bits, scale


def kernel_roofline(device, tokens: int, dim: int = D_MODEL, ffn: int = D_FFN) -> dict:
    """The dominant kernel alone: forward packed-sign GEMM of the up projection,
    [tokens, dim] x [ffn, dim]^T (4096 -> 14336 by default), bf16 in, fp32 accumulate, bf16 out."""

    from qste_b200 import kernels

    m, k, n = tokens, dim, ffn
    x, bits, scale = _gemm_inputs(device, m, k, n)
    for _ in range(3):
        kernels.packed_linear_affine(x, bits, scale, None, k)
    launches = 10
    seconds = timed(lambda: kernels.packed_linear_affine(x, bits, scale, None, k), launches) / launches
    flops = 2.0 * m * k * n
    peak = peaks()
    achieved = flops / seconds / 1e12
    return {"bound": "tensor", "kernel": "packed-sign forward GEMM", "shape": [m, k, n],
            "achieved": achieved, "peak": peak["bf16_tflops"], "unit": "TFLOP/s",
            "frac": achieved / peak["bf16_tflops"], "peak_source": peak["source"],
            # dram__bytes_read.sum + dram__bytes_write.sum of this kernel, one launch captured at the
            # bench's own 16384 tokens (profiles/packed_gemm_tc_three_products_16384x4096x14336.md:
            # 151.4 MB read + 449.7 MB written; algorithmic 611 MB, the last tiles of Y were still in
            # L2).  Other token counts: activations in and out scale with the tokens, the bits do not.
            "traffic": ((601.1e6 - 7.3e6) * m / 16384 + 7.3e6) if (k, n) == (D_MODEL, D_FFN) else None,
            "traffic_source": None if (k, n) != (D_MODEL, D_FFN) else
            "ncu capture of one launch at 16384 tokens" + ("" if m == 16384 else ", scaled by the token count"),
            "algorithmic_bytes": m * k * 2 + n * k / 8 + 4 * n + m * n * 2,
            "us_per_launch": seconds * 1e6}


def kernel_breakdown(device, tokens: int) -> dict:
    """Every kernel of the path at the workload's shapes, each timed alone."""

    from qste_b200 import kernels

    peak = peaks()
    m, k, n = tokens, D_MODEL, D_FFN
    x, bits, scale = _gemm_inputs(device, m, k, n)
    generator = torch.Generator(device=device).manual_seed(3)
    dy = torch.randn(m, n, device=device, dtype=torch.bfloat16, generator=generator)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x)
    aux = torch.stack((act_offset, act_scale))
    out = {}

    def gemm(name, fn, repeat=5):
        # each of these is compared with the burst peak: a pause lets the part leave the power cap
        # that the kernels timed before it drove it into
        torch.cuda.synchronize()
        time.sleep(2.0)
        fn()
        seconds = timed(fn, repeat) / repeat
        tflops = 2.0 * m * k * n / seconds / 1e12
        out[name] = {"us": seconds * 1e6, "tflops": tflops, "frac_tensor": tflops / peak["bf16_tflops"]}

    gemm("forward", lambda: kernels.packed_linear_affine(x, bits, scale, None, k))
    gemm("dx", lambda: kernels.packed_transpose(dy, bits, k, scale))
    gemm("evidence_fused", lambda: kernels.linear_backward_evidence(dy, act_bits, aux, k, bits, scale))
    bits.requires_grad_(False)
    torch.cuda.synchronize()
    time.sleep(2.0)
    kernels.linear_backward(dy, bits, scale, k, act_bits, aux)
    seconds = timed(lambda: kernels.linear_backward(dy, bits, scale, k, act_bits, aux), 5) / 5
    out["backward_whole"] = {"us": seconds * 1e6, "tflops": 4.0 * m * k * n / seconds / 1e12,
                             "frac_tensor": 4.0 * m * k * n / seconds / 1e12 / peak["bf16_tflops"]}

    def stream(name, fn, nbytes, repeat=5, replay=False):
        fn()
        timing = "calls"
        seconds = timed(fn, repeat) / repeat
        if replay:
            # a kernel of a few microseconds: the calls above are bound by the host side of a
            # call (wrapper, allocation, launch), so the same calls are also timed as one CUDA
            # graph replay, which leaves the kernels back to back on the device
            try:
                side = torch.cuda.Stream(device)
                side.wait_stream(torch.cuda.current_stream(device))
                with torch.cuda.stream(side):
                    fn()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        for _ in range(repeat):
                            fn()
                    graph.replay()
                    side.synchronize()
                    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    begin.record(side)
                    graph.replay()
                    end.record(side)
                    side.synchronize()
                out[name + "_calls_us"] = seconds * 1e6
                seconds = begin.elapsed_time(end) / 1e3 / repeat
                timing = "graph replay"
            except Exception as error:  # the per-call number stands
                out[name + "_replay_error"] = repr(error)[:200]
        gbs = nbytes / seconds / 1e9
        out[name] = {"us": seconds * 1e6, "gbs": gbs, "frac_hbm": gbs / peak["hbm_gbs"], "timing": timing}

    stream("pack_affine_rows", lambda: kernels.pack_affine_rows(x), m * k * 2 + m * k / 8 + 8 * m)
    coordinate = torch.randint(-127, 128, (n, k), device=device, dtype=torch.int8, generator=generator)
    stream("pack_coordinate", lambda: kernels.pack_coordinate(coordinate), n * k * 1.125)
    packed = kernels.pack_coordinate(coordinate)
    state = dict(moment_q=torch.zeros_like(coordinate),
                 moment_scale=torch.full((n * k // 256,), 1 / 127, dtype=torch.float16, device=device),
                 row_v=torch.zeros(n, dtype=torch.float16, device=device),
                 col_v=torch.zeros(k, dtype=torch.float16, device=device))
    evidence = torch.randn(n, k, device=device, generator=generator)
    scratch = torch.empty_like(evidence)
    flips = torch.zeros((), dtype=torch.int64, device=device)

    def update():
        scratch.copy_(evidence)
        kernels.coordinate_update(scratch, coordinate, packed, state["moment_q"], state["moment_scale"],
                                  state["row_v"], state["col_v"], beta1=0.9, beta2=0.99, update_clip=2.0,
                                  coordinate_lr=1.0, block_size=256, seed=1, step=0, flips=flips)

    copy_seconds = timed(lambda: scratch.copy_(evidence), 5) / 5
    update()
    seconds = timed(update, 5) / 5 - copy_seconds
    gbs = 8.125 * n * k / seconds / 1e9
    out["coordinate_update"] = {"us": seconds * 1e6, "gbs_compulsory": gbs, "frac_hbm": gbs / peak["hbm_gbs"],
                                "bytes_per_element_compulsory": 8.125}
    x1, bits1, scale1 = _gemm_inputs(device, 1, k, n, seed=4)
    stream("forward_m1_stream", lambda: kernels.packed_linear_affine(x1, bits1, scale1, None, k),
           n * k / 8 + 4 * n + 2 * k + 2 * n, repeat=20, replay=True)
    # 16 tokens: the register-expansion forward and the one-launch evidence (bits and result from L2
    # where they fit; `gemm_sweep` times the same calls over weight copies larger than L2)
    x16, bits16, scale16 = _gemm_inputs(device, 16, k, n, seed=5)
    stream("forward_m16_registers", lambda: kernels.packed_linear_affine(x16, bits16, scale16, None, k),
           n * k / 8 + 8 * n + 16 * (2 * k + 2 * n), repeat=20, replay=True)
    dy16 = torch.randn(16, n, device=device, dtype=torch.bfloat16, generator=generator)
    act16, offset16, ascale16 = kernels.pack_affine_rows(x16)
    aux16 = torch.stack((offset16, ascale16))
    stream("evidence_m16_tables", lambda: kernels.linear_backward_evidence(dy16, act16, aux16, k, bits16, scale16),
           4.0 * n * k + n * k / 8 + 16 * k / 8 + 2 * 16 * n + 12 * n, repeat=10)
    return out


# ------------------------------------------------------------------------------------------
# decoder workloads: the GPT-2-small and Llama-1.1B shapes with their MLPs converted
# (harness models in plain PyTorch: the reference ships none, only the training loop they plug into)
# ------------------------------------------------------------------------------------------

DECODERS = {
    # configs[2]: 12 layers, d = 768, 12 heads, MLP ratio 4, GELU, vocab 50257, seq 1024, batch 8, one GPU
    "gpt2_small": dict(layers=12, dim=768, heads=12, kv_heads=12, ffn=3072, mlp="gelu", norm="layer", rope=False,
                       vocab=50257, seq=1024, global_batch=8, micro_batch=8, tied_head=True,
                       include=["blocks.*.mlp.fc", "blocks.*.mlp.proj"]),
    # configs[3]: 22 layers, d = 2048, ffn 5632, 32 heads / 4 KV heads, RoPE, RMSNorm, vocab 32000, seq 2048,
    # global batch 64 sequences over the GPUs of the job (strong scaling)
    "llama_1b": dict(layers=22, dim=2048, heads=32, kv_heads=4, ffn=5632, mlp="swiglu", norm="rms", rope=True,
                     vocab=32000, seq=2048, global_batch=64, micro_batch=8, tied_head=False,
                     include=["blocks.*.mlp.gate", "blocks.*.mlp.up", "blocks.*.mlp.down"]),
}


class DecoderMLP(nn.Module):
    def __init__(self, spec, device):
        super().__init__()
        dim, ffn = spec["dim"], spec["ffn"]
        if spec["mlp"] == "swiglu":
            self.gate = nn.Linear(dim, ffn, bias=False, device=device)
            self.up = nn.Linear(dim, ffn, bias=False, device=device)
            self.down = nn.Linear(ffn, dim, bias=False, device=device)
            self.act = nn.SiLU()
        else:
            self.fc = nn.Linear(dim, ffn, device=device)
            self.proj = nn.Linear(ffn, dim, device=device)
            self.act = nn.GELU()
        self.gated = spec["mlp"] == "swiglu"

    def forward(self, x):
        if self.gated:
            return self.down(self.act(self.gate(x)) * self.up(x))
        return self.proj(self.act(self.fc(x)))


class DecoderAttention(nn.Module):
    def __init__(self, spec, device):
        super().__init__()
        dim, self.heads, self.kv_heads = spec["dim"], spec["heads"], spec["kv_heads"]
        self.head_dim = dim // self.heads
        bias = spec["norm"] == "layer"
        self.qkv = nn.Linear(dim, (self.heads + 2 * self.kv_heads) * self.head_dim, bias=bias, device=device)
        self.out = nn.Linear(dim, dim, bias=bias, device=device)
        self.rope = spec["rope"]

    def forward(self, x, rotary):
        batch, seq, _ = x.shape
        q, k, v = self.qkv(x).split([self.heads * self.head_dim, self.kv_heads * self.head_dim,
                                     self.kv_heads * self.head_dim], dim=-1)
        q = q.view(batch, seq, self.heads, self.head_dim).transpose(1, 2)
        k = k.view(batch, seq, self.kv_heads, self.head_dim).transpose(1, 2)
        v = v.view(batch, seq, self.kv_heads, self.head_dim).transpose(1, 2)
        if self.rope:
            cos, sin = rotary
            q = q * cos + torch.cat((-q[..., self.head_dim // 2:], q[..., : self.head_dim // 2]), -1) * sin
            k = k * cos + torch.cat((-k[..., self.head_dim // 2:], k[..., : self.head_dim // 2]), -1) * sin
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.heads != self.kv_heads)
        return self.out(y.transpose(1, 2).reshape(batch, seq, -1))


class DecoderBlock(nn.Module):
    def __init__(self, spec, device):
        super().__init__()
        make = (lambda: nn.LayerNorm(spec["dim"], device=device)) if spec["norm"] == "layer" \
            else (lambda: nn.RMSNorm(spec["dim"], device=device))
        self.norm1, self.norm2 = make(), make()
        self.attention = DecoderAttention(spec, device)
        self.mlp = DecoderMLP(spec, device)

    def forward(self, x, rotary):
        x = x + self.attention(self.norm1(x), rotary)
        return x + self.mlp(self.norm2(x))


class Decoder(nn.Module):
    def __init__(self, spec, device):
        super().__init__()
        self.spec = spec
        self.embed = nn.Embedding(spec["vocab"], spec["dim"], device=device)
        self.positions = None if spec["rope"] else nn.Embedding(spec["seq"], spec["dim"], device=device)
        self.blocks = nn.ModuleList([DecoderBlock(spec, device) for _ in range(spec["layers"])])
        self.norm = nn.LayerNorm(spec["dim"], device=device) if spec["norm"] == "layer" else nn.RMSNorm(spec["dim"], device=device)
        self.head = nn.Linear(spec["dim"], spec["vocab"], bias=False, device=device)
        if spec["tied_head"]:
            self.head.weight = self.embed.weight
        if spec["rope"]:
            half = spec["dim"] // spec["heads"] // 2
            frequency = 1.0 / (10000.0 ** (torch.arange(half, device=device, dtype=torch.float32) / half))
            angle = torch.outer(torch.arange(spec["seq"], device=device, dtype=torch.float32), frequency)
            angle = torch.cat((angle, angle), -1)
            self.register_buffer("cos", angle.cos()[None, None], persistent=False)
            self.register_buffer("sin", angle.sin()[None, None], persistent=False)

    def forward(self, ids):
        x = self.embed(ids)
        rotary = None
        if self.positions is not None:
            x = x + self.positions(torch.arange(ids.shape[1], device=ids.device))
        else:
            rotary = (self.cos[:, :, : ids.shape[1]].to(x.dtype), self.sin[:, :, : ids.shape[1]].to(x.dtype))
        for block in self.blocks:
            x = block(x, rotary)
        return self.head(self.norm(x))


def run_decoder(args) -> dict:
    """configs[2] / configs[3]: a decoder trained with only its MLPs converted.  One step = the
    job's global batch (forward, backward, AdamW on the float parameters, QSTEOptimizer on the
    coordinates); a rank whose share is more than one micro-batch of 8 sequences accumulates with
    `QSTEOptimizer.prepare_accumulation()` and applies the summed evidence once per step."""

    import qste_b200 as qste
    from qste_b200 import distributed as qdist
    from qste_b200 import kernels

    spec = DECODERS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    if spec["global_batch"] % world:
        raise SystemExit(f"{args.workload}: global batch {spec['global_batch']} does not divide over {world} GPUs")
    per_rank = spec["global_batch"] // world
    micro = min(spec["micro_batch"], per_rank)
    micro_steps = per_rank // micro
    seq = spec["seq"]

    torch.manual_seed(1234)
    model = Decoder(spec, device)
    qste.convert(model, include=spec["include"])
    reducer = qdist.mean_evidence(overlap=True, reserve_sms=args.reserve if args.reserve >= 0 else None) if world > 1 else None
    coordinates = qste.QSTEOptimizer(model, gradient_reducer=reducer if reducer else False, async_update=micro_steps == 1)
    if micro_steps > 1:
        coordinates.prepare_accumulation()
    floats = list(qste.continuous_parameters(model))
    host_optimizer = torch.optim.AdamW(floats, lr=1e-4, fused=True)
    wrapped = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel

        # float parameters (attention, norms, embeddings, row scales, biases) ride DDP's buckets; the
        # coordinate evidence is not an autograd gradient and goes through the evidence reducer
        wrapped = DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True)

    generator = torch.Generator().manual_seed(1000 + rank)
    pinned = [torch.randint(0, spec["vocab"], (per_rank, seq + 1), generator=generator).pin_memory() for _ in range(2)]
    resident = [batch.to(device) for batch in pinned]
    counter = {"step": 0, "flips": 0}

    def step(ids):
        total = None
        for index in range(micro_steps):
            chunk = ids[index * micro:(index + 1) * micro]
            last = index == micro_steps - 1
            context = wrapped.no_sync() if (world > 1 and not last) else nullcontext()
            with context:
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    logits = wrapped(chunk[:, :-1])
                loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), chunk[:, 1:].reshape(-1)) / micro_steps
                loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        host_optimizer.step()
        counter["flips"] += coordinates.step()
        host_optimizer.zero_grad(set_to_none=True)
        if micro_steps == 1:
            coordinates.zero_grad()
        counter["step"] += 1
        return total

    def resident_step():
        step(resident[counter["step"] % 2])

    def e2e_step():
        ids = pinned[counter["step"] % 2].to(device, non_blocking=True)
        return float(step(ids).item())

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        resident_step()
    barrier()
    launches_before = launch_count()
    with ClockSampler(local) as clocks:
        seconds = timed(resident_step, args.steps)
    launches = launch_count() - launches_before
    barrier()
    seconds = max_over_ranks(seconds, world, device)
    e2e_step()
    barrier()
    e2e_seconds = max_over_ranks(timed(e2e_step, args.steps), world, device)

    tokens_per_step = spec["global_batch"] * seq
    mlp_rows = micro * seq
    result = {
        "metric": METRIC, "value": tokens_per_step * args.steps / seconds, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * seconds / args.steps,
        "higher_is_better": True, "scaling": "strong" if spec["global_batch"] > spec["micro_batch"] else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
        "config": {"workload": f"{args.workload}: {spec['layers']} layers, d={spec['dim']}, ffn={spec['ffn']}, "
                               f"{spec['heads']}/{spec['kv_heads']} heads, vocab {spec['vocab']}, seq {seq}, global batch "
                               f"{spec['global_batch']} sequences, MLPs converted ({len(coordinates.surfaces)} surfaces), "
                               f"bf16 autocast",
                   "parallelism": f"dp{world}", "sequences_per_gpu": per_rank, "micro_batches_per_step": micro_steps,
                   "l2": "each step's activations exceed L2 many times over; two rotating token batches"},
        "e2e": {"value": tokens_per_step * args.steps / e2e_seconds, "unit": "tokens/s",
                "h2d_bytes_per_step": per_rank * (seq + 1) * 8, "d2h_bytes_per_step": 4},
        "gpu_launches": launches, "clocks": clocks.summary(),
        "flips_per_step": counter["flips"] / max(1, counter["step"]),
        "wait_timeouts": kernels.wait_timeouts(device), "ranks_agree": bool(qdist.surfaces_agree(model)),
    }
    if rank == 0 and not args.no_extras:
        torch.cuda.synchronize()
        time.sleep(3.0)
        result["roofline"] = kernel_roofline(device, mlp_rows, spec["dim"], spec["ffn"])
        if world == 1:
            result["cpu_baseline"] = decoder_cpu_baseline(spec, mlp_rows, tokens_per_step)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_decoder_reference(args) -> dict:
    """`--impl reference` for a decoder workload: the per-block CPU figure of decoder_cpu_baseline
    as the arm's line (the MLP blocks are the path; the rest of the model is not run on the CPU)."""

    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    try:
        torch.set_num_threads(max(torch.get_num_threads(), len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    spec = DECODERS[args.workload]
    mlp_rows = min(spec["micro_batch"], spec["global_batch"]) * spec["seq"]
    baseline = decoder_cpu_baseline(spec, mlp_rows, spec["global_batch"] * spec["seq"])
    return {"impl": "reference", "metric": METRIC, "value": baseline["value"], "unit": "tokens/s",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": 1, "warmup": 0,
            "ms_per_step": 1e3 * baseline["seconds_per_block_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: converted MLP blocks only, on the CPU; ms_per_step is ONE block at "
                                   f"{mlp_rows} tokens, value = tokens / ({spec['layers']} layers x block time)"},
            "cpu_baseline": baseline,
            "e2e": {"value": baseline["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def decoder_cpu_baseline(spec, mlp_rows: int, tokens_per_step: int) -> dict:
    """The reference's CPU kernels on ONE converted MLP block of the decoder at a micro-batch's
    full token count: forward, backward and the block's coordinate updates.  Attention, norms,
    embeddings and the head are not on the path and are not run, so tokens/s = tokens / (layers x
    block time) bounds the CPU's whole-model figure from above."""

    if spec["mlp"] == "swiglu":
        times, _, split, kind = cpu_block_steps(mlp_rows, 1, 0, dim=spec["dim"], ffn=spec["ffn"])
    else:
        times, split, kind = cpu_plain_mlp_steps(mlp_rows, spec["dim"], spec["ffn"])
    seconds = statistics.median(times)
    return {"value": mlp_rows / (seconds * spec["layers"]), "unit": "tokens/s", "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": kind,
            "sample": f"one converted MLP block (d={spec['dim']}, ffn={spec['ffn']}) x {mlp_rows} tokens, fp32, forward + "
                      f"backward + coordinate updates, 1 step; MLP blocks only (attention, embeddings and head are not "
                      f"run): tokens/s = tokens / ({spec['layers']} layers x block time), an upper bound for the CPU",
            "seconds_per_block_step": seconds, "seconds_by_call": {key: round(value, 3) for key, value in split.items()}}


def cpu_plain_mlp_steps(tokens: int, dim: int, ffn: int):
    """One fc -> GELU -> proj block on the CPU through the reference's kernels, one step."""

    k, kind = _cpu_kernels()
    generator = torch.Generator().manual_seed(6)
    clock: dict = {}
    fc = CpuBinaryLinear(k, ffn, dim, generator, 0, clock)
    proj = CpuBinaryLinear(k, dim, ffn, generator, 1, clock)
    x = torch.randn(tokens, dim, generator=generator)
    begin = time.perf_counter()
    h = fc.forward(x)
    a = F.gelu(h)
    y = proj.forward(a)
    dy = y * (2.0 / y.numel())
    da, _, _ = proj.backward(dy, 0)
    cdf = 0.5 * (1.0 + torch.erf(h * 0.7071067811865476))
    dh = da * (cdf + h * torch.exp(-0.5 * h * h) * 0.3989422804014327)
    fc.backward(dh, 0)
    seconds = time.perf_counter() - begin
    clock["harness_elementwise"] = seconds - sum(clock.values())
    return [seconds], dict(clock), kind


# ------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU kernels on this box's host cores
# ------------------------------------------------------------------------------------------

def _cpu_kernels():
    """(namespace, kind): the compiled reference if it was built, else the oracle port."""

    sys.path.insert(0, str(ROOT))
    try:
        from oracle import build_ref

        module = build_ref.load()
    except Exception:
        module = None
    if module is not None:
        return module, "reference"
    import numpy as np

    import oracle

    class Port:
        @staticmethod
        def pack_affine_rows(x):
            return tuple(torch.from_numpy(a) for a in oracle.pack_affine_rows(x))

        @staticmethod
        def packed_linear_affine(x, packed, scale, bias, columns):
            return torch.from_numpy(oracle.packed_linear_affine(x, packed, scale, bias, columns))

        @staticmethod
        def packed_transpose(x, packed, columns, row_scale=None):
            return torch.from_numpy(oracle.packed_transpose(x, packed, columns, row_scale))

        @staticmethod
        def evidence_from_packed(g, packed, columns, row_scale=None):
            return torch.from_numpy(oracle.evidence_from_packed(g, packed, columns, row_scale))

        @staticmethod
        def packed_row_inner(m, packed, columns):
            return torch.from_numpy(oracle.packed_row_inner(m, packed, columns))

        @staticmethod
        def coordinate_update(g, c, p, mq, ms, rv, cv, b1, b2, clip, lr, block, seed, step):
            return oracle.coordinate_update(np.ascontiguousarray(g.numpy()), c.numpy(), p.numpy(), mq.numpy(),
                                            ms.numpy(), rv.numpy(), cv.numpy(), beta1=b1, beta2=b2,
                                            update_clip=clip, coordinate_lr=lr, block_size=block, seed=seed, step=step)

        @staticmethod
        def pack_coordinate(c):
            return torch.from_numpy(oracle.pack_coordinate(c))

    return Port, "port"


class CpuBinaryLinear:
    """One converted Linear on the CPU through the reference's kernels, following
    src/qste/functional.py:153-194 and src/qste/optim.py:156-178 call for call.  `clock`
    collects the seconds spent per kind of call."""

    def __init__(self, k, rows, columns, generator, index, clock):
        self.k, self.rows, self.columns, self.index, self.clock = k, rows, columns, index, clock
        self.coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
        self.packed = k.pack_coordinate(self.coordinate)
        self.scale = torch.full((rows,), 0.02)
        blocks = (rows * columns + 255) // 256
        self.moment_q = torch.zeros(rows, columns, dtype=torch.int8)
        self.moment_scale = torch.full((blocks,), 1 / 127, dtype=torch.float16)
        self.row_v = torch.zeros(rows, dtype=torch.float16)
        self.col_v = torch.zeros(columns, dtype=torch.float16)

    def timed(self, kind, call, *args):
        begin = time.perf_counter()
        result = call(*args)
        self.clock[kind] = self.clock.get(kind, 0.0) + time.perf_counter() - begin
        return result

    def forward(self, x):
        y = self.timed("gemm", self.k.packed_linear_affine, x, self.packed, self.scale, None, self.columns)
        self.saved = self.timed("pack_affine_rows", self.k.pack_affine_rows, x)
        return y

    def backward(self, dy, step):
        bits, offset, act_scale = self.saved
        dx = self.timed("gemm", self.k.packed_transpose, dy, self.packed, self.columns, self.scale)
        evidence = self.timed("gemm", self.k.evidence_from_packed, dy, bits, self.columns, act_scale)
        begin = time.perf_counter()
        evidence.add_(torch.mv(dy.t(), offset).unsqueeze(1))
        g_scale = self.k.packed_row_inner(evidence, self.packed, self.columns)
        evidence.mul_(self.scale.unsqueeze(1))
        self.clock["evidence_epilogue"] = self.clock.get("evidence_epilogue", 0.0) + time.perf_counter() - begin
        flips = self.timed("coordinate_update", self.k.coordinate_update, evidence, self.coordinate, self.packed,
                           self.moment_q, self.moment_scale, self.row_v, self.col_v, 0.9, 0.99, 2.0, 1.0, 256,
                           1 + 1_000_003 * self.index, step)
        return dx, g_scale, int(flips)


def cpu_block_steps(tokens: int, steps: int, warmup: int, budget_s: float | None = None,
                    dim: int = D_MODEL, ffn: int = D_FFN):
    """Training steps of ONE SwiGLU block on the CPU (forward, backward, three coordinate
    updates), each timed.  Runs `warmup + steps` steps, or as many as finish inside `budget_s`
    seconds (at least one).  Returns (seconds of every timed step, steps discarded as warm-up,
    seconds per kind of call summed over the timed steps, kind)."""

    k, kind = _cpu_kernels()
    generator = torch.Generator().manual_seed(5)
    clock: dict = {}
    gate = CpuBinaryLinear(k, ffn, dim, generator, 0, clock)
    up = CpuBinaryLinear(k, ffn, dim, generator, 1, clock)
    down = CpuBinaryLinear(k, dim, ffn, generator, 2, clock)
    x = torch.randn(tokens, dim, generator=generator)
    times, clocks = [], []
    started = time.perf_counter()
    for number in range(warmup + steps):
        clock.clear()
        begin = time.perf_counter()
        h = F.rms_norm(x, (dim,))
        g, u = gate.forward(h), up.forward(h)
        s = torch.sigmoid(g)
        a = g * s
        y = x + down.forward(a * u)
        dy = y * (2.0 / y.numel())
        dmid, _, _ = down.backward(dy, number)
        du = dmid * a
        dg = dmid * u * (s * (1 + g * (1 - s)))
        up.backward(du, number)
        gate.backward(dg, number)
        seconds = time.perf_counter() - begin
        clock["harness_elementwise"] = seconds - sum(clock.values())
        times.append(seconds)
        clocks.append(dict(clock))
        spent = time.perf_counter() - started
        if budget_s is not None and spent + 1.2 * seconds > budget_s:
            break
    # the first step pays for first-touch page faults of several GB: it is the warm-up whenever
    # there is a second one
    discarded = min(warmup, len(times) - 1)
    times, clocks = times[discarded:], clocks[discarded:]
    split = {key: sum(c.get(key, 0.0) for c in clocks) / len(clocks) for key in clocks[0]}
    return times, discarded, split, kind


def cpu_baseline(tokens: int = TOKENS) -> dict:
    """The reference's CPU kernels on ONE SwiGLU block at the workload's full token count, one
    step, measured not extrapolated; tokens/s of the 8-block stack = tokens / (8 x block time)."""

    times, _, split, kind = cpu_block_steps(tokens, 1, 0)
    seconds = statistics.median(times)
    return {"value": tokens / (seconds * BLOCKS), "unit": "tokens/s", "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": kind,
            "sample": f"one SwiGLU block (d={D_MODEL}, ffn={D_FFN}) x {tokens} tokens (the workload's own count), fp32, "
                      f"forward + backward + 3 coordinate updates, 1 step; tokens/s = tokens / ({BLOCKS} blocks x block time)",
            "seconds_per_block_step": seconds,
            "seconds_by_call": {key: round(value, 3) for key, value in split.items()}}


def run_reference(args) -> dict:
    """The reference's own CPU kernels on the workload of the repo arm.

    A step of the 8-block stack is eight identical blocks, so ONE block is timed, at the
    config's full token count (the three coordinate updates of a block cost the same whatever
    the batch, so a smaller batch would understate the CPU's tokens/s), and the stack's
    tokens/s is tokens / (8 x block time).  A block step takes tens of seconds on the host
    cores: the arm runs the steps that fit its time budget (QSTE_BENCH_REFERENCE_BUDGET_S,
    default 150 s), at least one, and reports how many it timed in `steps`."""

    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    # torchrun sets OMP_NUM_THREADS=1 for its workers; this arm is the reference on all host cores
    try:
        torch.set_num_threads(max(torch.get_num_threads(), len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    tokens = args.tokens or TOKENS
    budget = float(os.environ.get("QSTE_BENCH_REFERENCE_BUDGET_S", "150"))
    times, discarded, split, kind = cpu_block_steps(tokens, max(1, args.steps), max(0, args.warmup), budget_s=budget)
    seconds = statistics.median(times)
    value = tokens / (seconds * BLOCKS)
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": len(times), "warmup": discarded,
        "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": 1e3 * seconds, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(stack_config(BLOCKS, tokens, 1),
                       cpu_sample=f"the CPU arm times ONE of the {BLOCKS} identical blocks per step, at the full {tokens} "
                                  f"tokens: ms_per_step is that block step (median of {len(times)} timed inside a "
                                  f"{budget:.0f} s budget) and value = tokens / ({BLOCKS} x block time)"),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"one SwiGLU block x {tokens} tokens per step, fp32, all host threads torch uses; "
                                   f"{len(times)} timed step(s) after {discarded} warm-up",
                         "seconds_per_block_step": seconds,
                         "seconds_by_call": {key: round(v, 3) for key, v in split.items()}},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# ------------------------------------------------------------------------------------------
# packed-sign GEMM sweep (forward and backward), one GPU
# ------------------------------------------------------------------------------------------

def graph_time(calls, replays: int = 5) -> float:
    """Seconds per call for a list of calls captured into ONE CUDA graph and replayed: removes
    the host's launch overhead, which dwarfs a microsecond-scale kernel."""

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for call in calls:
            call()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for call in calls:
            call()
    graph.replay()
    seconds = timed(graph.replay, replays)
    return seconds / (replays * len(calls))


def run_sweep(args) -> dict:
    """configs[1]: forward, dX and evidence at M in {1, 16, 128, 4096, 16384} x four (K, N).

    Large batches are timed call by call with CUDA events.  Batches <= 128 take microseconds,
    so they are captured into a CUDA graph of back-to-back launches, each launch reading a
    DIFFERENT copy of the packed weight (copies add up to > 160 MB, more than L2), and the graph
    is replayed: the figure is per-launch device time with the bits coming from HBM."""

    from qste_b200 import kernels

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    peak = peaks()
    rows = []
    total_flops = total_seconds = 0.0
    for k, n in SWEEP_SHAPES:
        bit_bytes = n * k // 8
        copies = max(2, -(-(160 << 20) // bit_bytes))
        generator = torch.Generator(device=device).manual_seed(2)
        weights = [torch.randint(0, 256, (n, k // 8), device=device, dtype=torch.uint8, generator=generator)
                   for _ in range(copies)]
        scale = torch.rand(n, device=device, generator=generator) * 0.04 + 0.01
        for m in SWEEP_BATCHES:
            x = torch.randn(m, k, device=device, dtype=torch.bfloat16, generator=generator)
            dy = torch.randn(m, n, device=device, dtype=torch.bfloat16, generator=generator)
            act_bits, act_offset, act_scale = kernels.pack_affine_rows(x)
            aux = torch.stack((act_offset, act_scale))
            entry = {"m": m, "k": k, "n": n}
            small = m <= 128
            makers = {
                "forward": lambda w: (lambda: kernels.packed_linear_affine(x, w, scale, None, k)),
                "dx": lambda w: (lambda: kernels.packed_transpose(dy, w, k, scale)),
                "evidence": lambda w: (lambda: kernels.linear_backward_evidence(dy, act_bits, aux, k, w, scale)),
            }
            for name, make in makers.items():
                if small and name != "evidence":
                    seconds = graph_time([make(w) for w in weights])
                else:
                    fn = make(weights[0])
                    for _ in range(max(3, args.warmup)):
                        fn()
                    repeat = max(args.steps, 3 if m >= 4096 else 10)
                    seconds = timed(fn, repeat) / repeat
                flops = 2.0 * m * k * n
                entry[name] = {"us": seconds * 1e6, "tflops": flops / seconds / 1e12}
                if m >= 4096:
                    entry[name]["frac_tensor"] = entry[name]["tflops"] / peak["bf16_tflops"]
                    total_flops += flops
                    total_seconds += seconds
            if small:
                # forward at small batch is bound by streaming the packed bits
                entry["forward"]["bits_gbs"] = bit_bytes / (entry["forward"]["us"] * 1e-6) / 1e9
                entry["forward"]["frac_hbm"] = entry["forward"]["bits_gbs"] / peak["hbm_gbs"]
                entry["forward"]["timing"] = f"CUDA graph of {copies} launches over {copies} weight copies"
            rows.append(entry)
    value = total_flops / total_seconds / 1e12
    best = max((r for r in rows if r["m"] >= 4096), key=lambda r: r["forward"]["tflops"])
    small = [r for r in rows if r["m"] <= 128]
    extras = {
        "roofline": {"bound": "tensor", "kernel": f"packed-sign forward GEMM, M={best['m']}, K={best['k']}, N={best['n']}",
                     "achieved": best["forward"]["tflops"], "peak": peak["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": best["forward"]["tflops"] / peak["bf16_tflops"], "peak_source": peak["source"], "traffic": None,
                     "small_batch_hbm": {f"m{r['m']}_k{r['k']}_n{r['n']}": round(r["forward"]["frac_hbm"], 4) for r in small}},
    }
    if not args.no_extras:
        extras["cpu_baseline"] = sweep_cpu_baseline()
    return {**extras, "metric": "packed_sign_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "packed-sign GEMM sweep, forward + dX + evidence, M in {1,16,128,4096,16384} x "
                                   "4 (K,N); value = flop-weighted mean over M >= 4096"},
            "frac_tensor_peak": value / peak["bf16_tflops"], "sweep": rows}


def sweep_cpu_baseline(repeats: int = 3) -> dict:
    """configs[1] on the CPU through the reference's kernels (fp32: the reference up-casts bf16
    on the CPU): forward, dX and evidence at every (K, N) for M in {1, 16, 128}, and at
    M in {4096, 16384} for (4096, 14336); median of `repeats`."""

    k_ref, kind = _cpu_kernels()
    rows = []
    generator = torch.Generator().manual_seed(2)
    for k, n in SWEEP_SHAPES:
        packed = torch.randint(0, 256, (n, k // 8), generator=generator, dtype=torch.int32).to(torch.uint8)
        scale = torch.rand(n, generator=generator) * 0.04 + 0.01
        for m in SWEEP_BATCHES:
            if m > 128 and (k, n) != (D_MODEL, D_FFN):
                continue
            x = torch.randn(m, k, generator=generator)
            dy = torch.randn(m, n, generator=generator)
            bits, _, act_scale = k_ref.pack_affine_rows(x)
            entry = {"m": m, "k": k, "n": n}
            for name, call in (("forward", lambda: k_ref.packed_linear_affine(x, packed, scale, None, k)),
                               ("dx", lambda: k_ref.packed_transpose(dy, packed, k, scale)),
                               ("evidence", lambda: k_ref.evidence_from_packed(dy, bits, k, act_scale))):
                times = []
                for _ in range(repeats):
                    begin = time.perf_counter()
                    call()
                    times.append(time.perf_counter() - begin)
                seconds = statistics.median(times)
                entry[name] = {"us": seconds * 1e6, "tflops": 2.0 * m * k * n / seconds / 1e12}
            rows.append(entry)
    large = [r for r in rows if r["m"] >= 4096]
    flops = sum(3 * 2.0 * r["m"] * r["k"] * r["n"] for r in large)
    seconds = sum((r["forward"]["us"] + r["dx"]["us"] + r["evidence"]["us"]) * 1e-6 for r in large)
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": kind,
            "sample": f"fp32, median of {repeats}: all four (K,N) at M in {{1,16,128}}; M in {{4096,16384}} at (4096,14336) "
                      "only; value = flop-weighted mean over those large-M rows",
            "rows": rows}


def run_layer(args) -> dict:
    """configs[0]: one converted Linear, R = C = 2048, batch 256, fp32.  A step is one forward,
    one backward with an N(0,1) upstream gradient, one QSTEOptimizer step and one AdamW step on
    the row scales and the bias; `--impl reference` runs the same step on the CPU through the
    reference's kernels.  Value = steps per second of the median step (at least ten are timed)."""

    import numpy as np

    rows = columns = 2048
    batch = 256
    steps = max(10, args.steps)
    generator = torch.Generator().manual_seed(1)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    x = torch.randn(batch, columns, generator=generator)
    dy = torch.randn(batch, rows, generator=generator)
    config = {"workload": "single converted Linear, R=C=2048, batch 256, fp32: forward + backward + QSTEOptimizer step + "
                          "AdamW step on scale and bias", "l2": "the step's 17 MB evidence and 4 MB state fit L2: a latency-bound case"}
    common = {"metric": "converted_linear_steps_per_s", "unit": "steps/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
              "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
              "config": config}
    if args.impl == "reference":
        k_ref, kind = _cpu_kernels()
        clock: dict = {}
        layer = CpuBinaryLinear(k_ref, rows, columns, generator, 0, clock)
        layer.coordinate.copy_(coordinate)
        layer.packed = k_ref.pack_coordinate(layer.coordinate)
        log_scale = torch.full((rows,), float(np.log(0.02)), requires_grad=True)
        bias = torch.zeros(rows, requires_grad=True)
        host = torch.optim.AdamW([log_scale, bias], lr=1e-3)
        times = []
        for number in range(args.warmup + steps):
            begin = time.perf_counter()
            layer.scale = log_scale.detach().exp()
            y = layer.forward(x) + bias.detach()
            _, g_scale, _ = layer.backward(dy, number)
            log_scale.grad = g_scale * layer.scale
            bias.grad = dy.sum(0)
            host.step()
            if number >= args.warmup:
                times.append(time.perf_counter() - begin)
        seconds = statistics.median(times)
        del y
        return dict(common, impl="reference", value=1.0 / seconds, ms_per_step=1e3 * seconds,
                    cpu_baseline={"value": 1.0 / seconds, "unit": "steps/s", "cores": torch.get_num_threads(), "kind": kind,
                                  "sample": f"the whole step, median of {steps}"},
                    e2e={"value": 1.0 / seconds, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})

    import qste_b200 as qste

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    surface = qste.Surface(torch.zeros(rows, columns)).to(device)
    with torch.no_grad():
        surface.coordinate.copy_(coordinate)
        surface.refresh_packed()
        surface.log_scale.fill_(float(np.log(0.02)))
    layer = qste.QSTELinear(surface, torch.zeros(rows)).to(device)
    coordinates = qste.QSTEOptimizer([surface])
    host = torch.optim.AdamW(list(layer.parameters()), lr=1e-3, fused=True)
    xd, dyd = x.to(device), dy.to(device)
    x_pinned, dy_pinned = x.pin_memory(), dy.pin_memory()

    def step(inputs, upstream):
        layer(inputs).backward(upstream)
        host.step()
        flips = coordinates.step()
        host.zero_grad(set_to_none=True)
        coordinates.zero_grad()
        return flips

    def timed_steps(fn):
        times = []
        for number in range(args.warmup + steps):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            if number >= args.warmup:
                times.append(begin.elapsed_time(end) / 1e3)
        return statistics.median(times)

    launches_before = launch_count()
    with ClockSampler(0) as clocks:
        seconds = timed_steps(lambda: step(xd, dyd))
    launches = (launch_count() - launches_before) * steps // (args.warmup + steps)
    e2e_seconds = timed_steps(lambda: step(x_pinned.to(device, non_blocking=True), dy_pinned.to(device, non_blocking=True)))
    result = dict(common, value=1.0 / seconds, ms_per_step=1e3 * seconds, gpu_launches=launches, clocks=clocks.summary(),
                  e2e={"value": 1.0 / e2e_seconds, "unit": "steps/s", "h2d_bytes_per_step": (x.numel() + dy.numel()) * 4,
                       "d2h_bytes_per_step": 8})
    # the step's dominant kernel by bytes: the coordinate update of 4.2 M coordinates
    from qste_b200 import kernels

    state = coordinates.state[id(surface)]
    evidence = torch.randn(rows, columns, device=device)
    scratch = torch.empty_like(evidence)
    flips = torch.zeros((), dtype=torch.int64, device=device)

    def update():
        scratch.copy_(evidence)
        kernels.coordinate_update(scratch, surface.coordinate.data, surface.packed_sign.data, state["moment_q"],
                                  state["moment_scale"], state["row_v"], state["col_v"], beta1=0.9, beta2=0.99,
                                  update_clip=2.0, coordinate_lr=1.0, block_size=256, seed=1, step=0, flips=flips)

    update()
    copy_seconds = timed(lambda: scratch.copy_(evidence), 20) / 20
    update_seconds = timed(update, 20) / 20 - copy_seconds
    peak = peaks()
    achieved = 8.125 * rows * columns / update_seconds / 1e9
    result["roofline"] = {"bound": "hbm", "kernel": "coordinate_update (9 launches), 2048 x 2048", "achieved": achieved,
                          "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"],
                          "peak_source": peak["source"], "traffic": None, "us_per_launch": update_seconds * 1e6,
                          "note": "compulsory bytes (8.125 per coordinate) over the time of the whole update; at this "
                                  "size the state fits L2 and the nine dependent launches bound it, not DRAM"}
    if not args.no_extras:
        reference = run_layer(argparse.Namespace(**{**vars(args), "impl": "reference"}))
        result["cpu_baseline"] = dict(reference["cpu_baseline"], ms_per_step=reference["ms_per_step"])
    return result


def run_kernel(args) -> dict:
    """One kernel of the path, launched `steps` times after `warmup` (for profiling)."""

    from qste_b200 import kernels

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    m, k, n = args.tokens or TOKENS, D_MODEL, D_FFN
    x, bits, scale = _gemm_inputs(device, m, k, n)
    generator = torch.Generator(device=device).manual_seed(3)
    if args.kernel in ("dx", "evidence", "backward"):
        dy = torch.randn(m, n, device=device, dtype=torch.bfloat16, generator=generator)
        act_bits, act_offset, act_scale = kernels.pack_affine_rows(x)
        aux = torch.stack((act_offset, act_scale))
    if args.kernel in ("update", "pack_coordinate", "row_inner"):
        coordinate = torch.randint(-127, 128, (n, k), device=device, dtype=torch.int8, generator=generator)
        packed = kernels.pack_coordinate(coordinate)
        moment_q = torch.zeros_like(coordinate)
        moment_scale = torch.full((n * k // 256,), 1 / 127, dtype=torch.float16, device=device)
        row_v = torch.zeros(n, dtype=torch.float16, device=device)
        col_v = torch.zeros(k, dtype=torch.float16, device=device)
        evidence = torch.randn(n, k, device=device, generator=generator)
        flips = torch.zeros((), dtype=torch.int64, device=device)
    calls = {
        "forward": lambda: kernels.packed_linear_affine(x, bits, scale, None, k),
        "dx": lambda: kernels.packed_transpose(dy, bits, k, scale),
        "evidence": lambda: kernels.linear_backward_evidence(dy, act_bits, aux, k, bits, scale),
        "backward": lambda: kernels.linear_backward(dy, bits, scale, k, act_bits, aux),
        "pack": lambda: kernels.pack_affine_rows(x),
        "pack_coordinate": lambda: kernels.pack_coordinate(coordinate),
        "row_inner": lambda: kernels.packed_row_inner(evidence, packed, k),
        "update": lambda: kernels.coordinate_update(
            evidence, coordinate, packed, moment_q, moment_scale, row_v, col_v, beta1=0.9, beta2=0.99,
            update_clip=2.0, coordinate_lr=1.0, block_size=256, seed=1, step=0, flips=flips),
    }
    call = calls[args.kernel]
    for _ in range(args.warmup):
        call()
    seconds = timed(call, args.steps) / args.steps
    return {"kernel": args.kernel, "shape": [m, k, n], "us": seconds * 1e6,
            "tflops": 2.0 * m * k * n / seconds / 1e12 if args.kernel in ("forward", "dx", "evidence") else None}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="mlp_stack",
                        choices=["mlp_stack", "gemm_sweep", "layer_2048", "gpt2_small", "llama_1b", "kernel"])
    parser.add_argument("--kernel", default="forward", choices=["forward", "dx", "evidence", "backward", "pack", "pack_coordinate", "row_inner", "update"],
                        help="with --workload kernel: which kernel to launch")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the per-kernel roofline section and the CPU baseline (profiling runs)")
    parser.add_argument("--trace", action="store_true",
                        help="mlp_stack on one GPU: add a profiler-based account of where a step's time goes")
    parser.add_argument("--tokens", type=int, default=0, help="tokens per GPU (default 16384)")
    parser.add_argument("--reserve", type=int, default=-1,
                        help="SMs the backward GEMMs leave to the all-reduce at N > 1 (default: the library's, 8)")
    parser.add_argument("--blocks", type=int, default=0, help="SwiGLU blocks (default 8)")
    args = parser.parse_args()
    if args.workload == "layer_2048":
        result = run_layer(args)
    elif args.impl == "reference" and args.workload in DECODERS:
        result = run_decoder_reference(args)
    elif args.impl == "reference" and args.workload == "gemm_sweep":
        baseline = sweep_cpu_baseline() if int(os.environ.get("RANK", "0")) == 0 else None
        result = {} if baseline is None else {
            "impl": "reference", "metric": "packed_sign_gemm_tflops", "value": baseline["value"], "unit": "TFLOP/s",
            "n_gpus": 1, "steps": 3, "warmup": 0, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": "packed-sign GEMM sweep on the CPU: " + baseline["sample"]},
            "cpu_baseline": baseline,
            "e2e": {"value": baseline["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    elif args.impl == "reference":
        result = run_reference(args)
    elif args.workload == "gemm_sweep":
        result = run_sweep(args)
    elif args.workload == "kernel":
        result = run_kernel(args)
    elif args.workload in DECODERS:
        result = run_decoder(args)
    else:
        result = run_ours(args)
    if result:
        print(json.dumps(result))


if __name__ == "__main__":
    main()

"""MoE layer forward+backward benchmark (tokens/s) on B200, with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: one MoE layer fwd+bwd at T=8192, d=4096, 64 experts, top-8, ffn 1408 (bf16 weights N(0,0.02),
activations / upstream gradient N(0,1), fp32 router logits from a bf16 router weight); synthetic seeded data.
The line also carries `ns_shape`: the same layer at T=32768 on the one GPU (device-timed, with its GEMM fractions),
`block_ops`: the bandwidth-bound ops of the block around the MoE feed-forward and of the head, and attention, each
against its own bound, and `decoder_step`: the full training step of the 16-layer MoE decoder configuration
(forward, backward, AdamW; tokens/s).
N > 1 (launched with torch.distributed.run, one rank per GPU): the expert-parallel layer, 64 experts sharded
over the ranks, T=32768 tokens per GPU (weak scaling); rows travel over NVLink peer memory, out through the gather
kernel and back through the epilogue of the last GEMM of each pass (B200_EP_TRANSPORT=fused|c|p2p|nccl; `c_driver` is
the same step through the C entry points b200_ep_moe_block_fwd / _bwd, timed after the main region). After the
timed regions every rank runs one small expert-parallel layer against the CPU oracle (`ep_parity`; a mismatch
replaces the line by an error and exit code 1), and rank 0 runs the same per-GPU batch on one GPU with all experts
(`same_batch_1gpu`), from which `efficiency_same_batch` = value / (N x that value).

Prints ONE JSON line on rank 0. `value` is device-timed with inputs resident in HBM; `e2e` is the same step
driven from pinned host buffers with the host<->device copies inside the timed region (`host_link` gives what the
host path delivers per GPU for those copies alone); `roofline` covers the grouped tcgen05 GEMM launches (the dominant
kernel) and `kernels` lists every op group with its own bound; `cpu_baseline` is the CPU oracle timed on a bounded
token sample of the same shape, and on the CPU-runnable configuration (T=2048, d=1024, 16 experts, top-2) in full,
on this box's host cores.
`--block-ops` prints only the block / head ops record (one launch of each kernel per repetition, for profiler
captures); with `--attention` the fused attention forward and backward too.
`--impl reference` times that CPU restatement of the reference's algorithm only (the reference has no CPU
implementation of this path of its own, and its CUDA kernels are what this repository replaces); under
torch.distributed.run rank 0 alone runs it, on all host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_layer_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
CFG_1GPU = dict(T=8192, d=4096, E=64, k=8, f=1408)       # the 1-GPU configuration the metric is quoted on
CFG_NS = dict(T=32768, d=4096, E=64, k=8, f=1408)        # the target shape: T=32768 on one GPU
CFG_EP = dict(T=32768, d=4096, E=64, k=8, f=1408)        # expert-parallel configuration, T per GPU
CFG_CPU_FULL = dict(T=2048, d=1024, E=16, k=2, f=1024)   # the CPU-runnable configuration, run in full on the host
CPU_SAMPLE_TOKENS = 1024


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, power = [], set(), []
        smax = None
        try:
            with open(self.path) as fh:
                for line in fh:
                    parts = [x.strip() for x in line.split(",")]
                    if len(parts) < 8:
                        continue
                    try:
                        clocks.append(float(parts[0]))
                        smax = float(parts[1])
                        power.append(float(parts[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         parts[4:8]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
        finally:
            os.unlink(self.path)
        if clocks:
            # samples taken while the GPU was busy: the upper half of the power readings
            busy = sorted(c for c, p in zip(clocks, power) if p >= 0.5 * max(power)) or sorted(clocks)
            out.update(sm_mhz=busy[len(busy) // 2], sm_max_mhz=smax, reasons=sorted(reasons), samples=len(clocks),
                       power_w_max=max(power))
        return out


# ------------------------------------------------------------------------------------------ block ops
# rows: 8 sequences of the training step's 8192 tokens, so that every tensor of an op is larger than L2
CFG_BLOCK = dict(T=65536, d=2048, heads=16, kv_heads=4, head_dim=128, vocab=128256, theta=500000)


def block_ops_profile(dev, peaks, iters=5, with_attention=True):
    """The bandwidth-bound ops around the MoE feed-forward at the row shapes of the decoder training step (d=2048,
    16 query / 4 kv heads of 128, vocabulary 128256) over 65536 token rows (inputs larger than L2): ms per launch
    (CUDA events, L2 flushed before each launch) and algorithmic bytes / time against the measured HBM rate."""
    import torch

    from ml_dataflow_b200 import ops

    c = CFG_BLOCK
    T, d, V = c["T"], c["d"], c["vocab"]
    kvd = c["kv_heads"] * c["head_dim"]
    g = torch.Generator(device=dev).manual_seed(11)
    bf = lambda shape, std=1.0: (torch.randn(shape, generator=g, device=dev) * std).to(torch.bfloat16)
    X, up, dX, w = bf((T, d)), bf((T, d)), bf((T, d)), bf((d,))
    out = torch.empty_like(X)
    rms = torch.empty(T, dtype=torch.float32, device=dev)
    dW = torch.zeros(d, dtype=torch.bfloat16, device=dev)
    ws = torch.empty(ops.rms_norm_bwd_w_workspace_bytes(T, d), dtype=torch.uint8, device=dev)
    q, kk = bf((T, d)), bf((T, kvd))
    pos = (torch.arange(T, dtype=torch.int32, device=dev) % 8192).contiguous()
    rows_sm = 2048  # softmax on a slice of the token rows: 2048 x 128256 bf16 = 0.5 GB each way
    logits = bf((rows_sm, V), 2.0)
    probs = torch.empty_like(logits)
    labels = torch.randint(0, V, (rows_sm,), generator=g, device=dev, dtype=torch.int32)
    loss = torch.zeros(rows_sm + 1, dtype=torch.float32, device=dev)
    n_par = 64 << 20
    par, grad, mean = bf((n_par,), 0.02), bf((n_par,), 0.01), bf((n_par,), 0.01)
    var = bf((n_par,), 0.01).abs()
    ids = torch.randint(0, V, (T,), generator=g, device=dev, dtype=torch.int64)
    sorted_ids, order = torch.sort(ids, stable=True)
    first = torch.ones(T, dtype=torch.bool, device=dev)
    first[1:] = sorted_ids[1:] != sorted_ids[:-1]
    starts = torch.cat([torch.nonzero(first).flatten(), torch.tensor([T], device=dev)]).to(torch.int32)
    nu = int(starts.numel()) - 1
    sid32, map32 = sorted_ids.to(torch.int32), order.to(torch.int32)
    table = bf((V, d), 0.02)
    gtab = torch.zeros_like(table)
    emb = torch.empty((T, d), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ops.rms_norm(T, d, 1e-5, w, X, out, rms)
    cases = [
        ("rms_norm", lambda: ops.rms_norm(T, d, 1e-5, w, X, out, rms), 4 * T * d),
        ("rms_norm_bwd_x", lambda: ops.rms_norm_bwd_x(T, d, 1e-5, rms, w, X, up, dX, None), 8 * T * d),
        ("rms_norm_bwd_w", lambda: ops.rms_norm_bwd_w(T, d, 1e-5, rms, X, up, dW, ws), 4 * T * d),
        ("rope", lambda: ops.rope(T, d, c["head_dim"], c["kv_heads"], c["theta"], pos, q, kk), 4 * T * (d + kvd)),
        ("softmax", lambda: ops.softmax(rows_sm, V, logits, probs), 4 * rows_sm * V),
        ("adamw_step", lambda: ops.adamw_step(n_par, 1, 3e-4, 0.9, 0.95, 0.1, 1e-8, par, grad, mean, var), 14 * n_par),
        ("embedding_table", lambda: ops.embedding_table(nu, d, sid32, map32, starts, table, emb), 2 * nu * d + 2 * T * d),
        ("embedding_table_bwd_w", lambda: ops.embedding_table_bwd_w(nu, d, sid32, map32, starts, up, gtab),
         2 * T * d + 4 * nu * d),
    ]
    res = {}
    for name, fn, nbytes in cases:
        fn()
        ms = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        t = sorted(ms)[len(ms) // 2]
        gbs = nbytes / (t * 1e-3) / 1e9
        res[name] = dict(ms=round(t, 4), bound="hbm", achieved=round(gbs, 1), unit="GB/s", frac=round(gbs / peaks["hbm_gbs"], 4))
    # attention at the decoder step's shape: one sequence of 8192 tokens, 16 query / 4 key-value heads of 128, causal.
    # Useful flop: two products over the visible half of the score matrix forward, five backward.
    del X, up, dX, out, q, kk, par, grad, mean, var, table, gtab, emb
    torch.cuda.empty_cache()
    if not with_attention:
        return res
    Ta, Hq, Hkv, hd = 8192, c["heads"], c["kv_heads"], c["head_dim"]
    aq, ak, av = bf((Ta, Hq * hd)), bf((Ta, Hkv * hd)), bf((Ta, Hkv * hd))
    ao, ado = torch.empty_like(aq), bf((Ta, Hq * hd))
    adq, adk, adv = torch.empty_like(aq), torch.empty_like(ak), torch.empty_like(av)
    alse = torch.empty((Hq, Ta), dtype=torch.float32, device=dev)
    aws = torch.empty(ops.attention_workspace_bytes(True, Hq, Hkv, hd, Ta, Ta, Ta), dtype=torch.uint8, device=dev)
    fwd_flop = 2 * 2 * Ta * Ta * hd * Hq / 2
    for name, fn, flop in (
            ("attention_fwd", lambda: ops.attention_fwd([0], [Ta], [0], [Ta], Hq, Hkv, hd, aq, ak, av, ao, alse, True, aws), fwd_flop),
            ("attention_bwd", lambda: ops.attention_bwd([0], [Ta], [0], [Ta], Hq, Hkv, hd, aq, ak, av, ao, alse, ado, adq, adk,
                                                        adv, True, aws), 2.5 * fwd_flop)):
        fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / 3
        tf = flop / (t * 1e-3) / 1e12
        res[name] = dict(ms=round(t, 3), bound="tensor", achieved=round(tf, 1), unit="TFLOP/s (causal half only)",
                         frac=round(tf / peaks["bf16_tflops"], 4),
                         note="fused tcgen05 kernels (scores and probabilities stay on the SM); flop counted over the visible half of "
                              "the score matrix only")
    del aq, ak, av, ao, ado, adq, adk, adv, alse, aws
    # one thread per row, one element each: a latency measurement, not a bandwidth one
    ops.cross_entropy_loss(rows_sm, V, probs, labels, loss)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    ops.cross_entropy_loss(rows_sm, V, probs, labels, loss)
    ops.set_average_loss(rows_sm, loss)
    e1.record()
    torch.cuda.synchronize()
    res["cross_entropy_loss+set_average_loss"] = dict(ms=round(e0.elapsed_time(e1), 4), bound="latency", rows=rows_sm)
    res["shapes"] = ("65536 token rows x d 2048 (norm, rope with 16q/4kv heads of 128, embedding over a 128256-row table), "
                     "softmax on 2048 x 128256 logits, AdamW on 64 Mi parameters; median of %d launches, L2 flushed "
                     "before each; attention: one causal sequence of 8192 tokens, 16 query / 4 kv heads of 128" % iters)
    return res


# ------------------------------------------------------------------------------------------ decoder step
def decoder_step_run(dev, peaks, steps=3, warmup=2):
    """The full training step of the 16-layer decoder configuration on one GPU: a random-init MoE decoder (16 layers, d=2048, 16 query /
    4 kv heads of 128, 64 experts top-8 with ffn 1024, vocabulary 128256, untied embeddings), one sequence of 8192 tokens
    with token ids and labels uniform over the vocabulary, bf16 parameters and gradients, AdamW (lr 3e-4, betas
    0.9 / 0.95, weight decay 0.1): forward + backward + optimizer step through ml_dataflow_b200.decoder, device-timed."""
    import torch

    from ml_dataflow_b200.decoder import Decoder, DecoderConfig

    cfg = DecoderConfig(n_layers=16, d=2048, n_heads=16, n_kv_heads=4, head_dim=128, n_experts=64, top_k=8, ffn=1024,
                        vocab=128256, eps=1e-5, theta=500000)
    T = 8192
    dec = Decoder(cfg, T, T, device=dev, seed=1)
    g = torch.Generator(device=dev).manual_seed(2)
    tokens = torch.randint(0, cfg.vocab, (T,), generator=g, device=dev, dtype=torch.int32)
    labels = torch.randint(0, cfg.vocab, (T,), generator=g, device=dev, dtype=torch.int32)

    def step():
        dec.zero_grads()
        loss = dec.forward(tokens, labels, [T])
        dec.backward()
        dec.adamw_step(lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1)
        return loss.clone()  # the returned scalar is a view of the loss buffer the next step overwrites

    losses = []
    for _ in range(warmup):
        losses.append(step())
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        losses.append(step())
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    losses = [float(x.item()) for x in losses]
    flop = dec.flops_per_token() * T
    rec = dict(workload="MoE decoder training step: 16 layers, d=2048, 16q/4kv heads of 128, 64 experts top-8 ffn 1024, "
                        "vocab 128256, 1 x 8192 tokens, bf16, AdamW", ms_per_step=round(ms, 2),
               value=round(T / (ms * 1e-3), 1), unit="tokens/s", steps=steps, warmup=warmup,
               parameters=dec.num_params(), matmul_tflops=round(flop / (ms * 1e-3) / 1e12, 1),
               matmul_frac_of_burst_peak=round(flop / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4),
               loss_per_step=[round(x, 4) for x in losses],
               note="the same batch every step, so the loss falls from ln(vocab) + 0.4 as the model memorises it; matmul "
                    "flop = 6 per active weight and token, attention excluded")
    del dec
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_reference_run(cfg, tokens, steps, warmup):
    """Times the CPU oracle (fwd+bwd) on `tokens` tokens of the shape `cfg`, on every host core this process may use.
    Returns (tokens/s, seconds per pass, threads)."""
    import numpy as np
    from oracle import oracle as orc

    orc.build()
    threads = orc.use_all_cores()  # process launchers export OMP_NUM_THREADS=1
    Ts, d, E, k, f = tokens, cfg["d"], cfg["E"], cfg["k"], cfg["f"]
    X, dOut = orc.normal_bf16((Ts, d), 0xB2000001), orc.normal_bf16((Ts, d), 0xB2000002)
    Wr = orc.normal_bf16((E, d), 0xB2000003, std=0.02)
    W1 = orc.normal_bf16((E, f, d), 0xB2000004, std=0.02)
    W3 = orc.normal_bf16((E, f, d), 0xB2000005, std=0.02)
    W2 = orc.normal_bf16((E, d, f), 0xB2000006, std=0.02)
    grads = dict(dW1=np.zeros_like(W1), dW3=np.zeros_like(W3), dW2=np.zeros_like(W2), dWr=np.zeros_like(Wr))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        fwd = orc.moe_forward(X, Wr, W1, W3, W2, k)
        orc.moe_backward(X, Wr, W1, W3, W2, k, fwd, dOut, grads=grads)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return Ts / sec, sec, threads


def cpu_baseline_record(cfg, steps, warmup):
    """The CPU legs: a bounded token sample of the workload `cfg` (the value that sits beside the GPU number) and the
    CPU-runnable configuration in full."""
    tps, sec, threads = cpu_reference_run(cfg, CPU_SAMPLE_TOKENS, steps, warmup)
    full_tps, full_sec, _ = cpu_reference_run(CFG_CPU_FULL, CFG_CPU_FULL["T"], 2, 1)
    c = CFG_CPU_FULL
    return dict(
        value=tps, unit=UNIT, cores=threads, kind="port",
        sample=(f"{CPU_SAMPLE_TOKENS} tokens of the workload shape (d={cfg['d']}, E={cfg['E']}, top-{cfg['k']}, ffn "
                f"{cfg['f']}), fwd+bwd through the CPU restatement of the reference kernels, OpenMP, {sec:.1f} s per pass"),
        cpu_config_in_full=dict(workload=workload_name(c, 1), value=full_tps, unit=UNIT, ms_per_step=full_sec * 1e3,
                                steps=2, warmup=1)), sec


def run_reference_arm(args, cfg, world):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # one sample pass costs a few seconds of CPU: the step count is bounded so the run ends within minutes
    steps, warmup = min(max(1, args.steps), 3), min(max(0, args.warmup), 1)
    rec, sec = cpu_baseline_record(cfg, steps, warmup)
    line = dict(metric=METRIC, value=rec["value"], unit=UNIT, n_gpus=world, steps=steps, warmup=warmup,
                steps_requested=args.steps, warmup_requested=args.warmup, ms_per_step=sec * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic", impl="reference",
                config=dict(workload=workload_name(cfg, world), T_sample=CPU_SAMPLE_TOKENS),
                cpu_baseline=rec,
                e2e=dict(value=rec["value"], unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line), flush=True)


def workload_name(cfg, world):
    base = f"moe_layer_fwd_bwd T={cfg['T']} d={cfg['d']} E={cfg['E']} top{cfg['k']} ffn={cfg['f']}"
    return base + (f" expert-parallel x{world} (T per GPU)" if world > 1 else "")


# ------------------------------------------------------------------------------------------ GPU arm
def algorithmic_work(cfg):
    """Algorithmic bytes / flops of each op group for one step (R = T*k routed rows, bf16 = 2 B)."""
    T, d, E, k, f = cfg["T"], cfg["d"], cfg["E"], cfg["k"], cfg["f"]
    R = T * k
    gather = 2 * T * d + 2 * R * d + 4 * R
    combine = 2 * R * d + 4 * T * d + 8 * R
    return {
        "router_gemm": ("hbm", 2 * T * d + 2 * E * d + 4 * T * E),
        "select_experts": ("hbm", 4 * T * E + 6 * T * k),
        "build_expert_mapping": ("hbm", 2 * T * k + 8 * T * k),
        "prepare_experts": ("hbm", gather),
        "experts_fwd_gemm": ("tensor", 6 * R * d * f),
        "merge_experts": ("hbm", combine),
        "prepare_experts_weighted": ("hbm", gather + 4 * R),
        "experts_bwd_x_gemm": ("tensor", 6 * R * d * f),
        "experts_bwd_w_gemm": ("tensor", 6 * R * d * f),
        "unpermute": ("hbm", 2 * R * d + 2 * T * d + 4 * R),  # one pass that overwrites dXn: no read of the output
        "router_grad": ("hbm", 4 * R + 2 * T * E * 3 + 4 * T * d + 2 * T * d + 4 * E * d),
    }


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the seven expert GEMM launches of one step, from an
# ncu pass over the same workload. It is a recorded profile figure, not a measurement of the present run.
NCU_GEMM_DRAM_BYTES_PER_STEP = {(8192, 4096, 64, 8, 1408): 16.5e9}
NCU_TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum over the 7 launches of one step, one pass, "
                      "recorded from a profiler run of this workload (not measured by this run)")

NVLINK_PEER_GBS_RECORDED = 770.0  # peer copy per direction recorded for this machine type (nominal 900)


def exchange_work(cfg, world):
    """Bytes each rank sends (and receives) per exchange when rows spread evenly over the ranks."""
    R = cfg["T"] * cfg["k"]
    rows = 2 * R * cfg["d"] * (world - 1) / world
    return {"dispatch": rows, "return": rows, "dispatch_bwd": rows, "return_bwd": rows + 4 * R * (world - 1) / world}


def gpu_numa_cpus(index):
    """(numa node, cpu list) of the GPU `index`, read from sysfs; (None, None) when it cannot be told."""
    try:
        import torch

        pr = torch.cuda.get_device_properties(index)
        addr = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{addr}/numa_node") as fh:
            node = int(fh.read().strip())
        if node < 0:
            return None, None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus = set()
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        return node, cpus
    except Exception:
        return None, None


def per_op_profile(layer, step, work, peaks, reps):
    """Runs `step` with an event between the ops and returns ({group: record}, GEMM ms, GEMM flop, raw ms per mark)."""
    import torch

    acc = {}
    for it in range(reps + 1):
        layer.profile = []
        step()
        layer.mark("end")
        torch.cuda.synchronize()
        marks = layer.profile
        layer.profile = None
        if it == 0:
            continue  # the first marked step may set up communicators the timed path never used
        per_step = {}  # a phase that runs in slices is marked once per slice: sum inside the step
        for (name, ev), (_, nxt) in zip(marks[:-1], marks[1:]):
            per_step[name] = per_step.get(name, 0.0) + ev.elapsed_time(nxt)
        for name, ms in per_step.items():
            acc.setdefault(name, []).append(ms)
    kernels = {}
    gemm_ms, gemm_flops = 0.0, 0
    for name, (bound, amount) in work.items():
        if name not in acc:
            continue
        ms = sum(acc[name]) / len(acc[name])
        if bound == "tensor":
            ach = amount / (ms * 1e-3) / 1e12
            kernels[name] = dict(ms=round(ms, 4), bound="tensor", achieved=round(ach, 1), unit="TFLOP/s",
                                 frac=round(ach / peaks["bf16_tflops_sustained"], 4),
                                 frac_of_burst_peak=round(ach / peaks["bf16_tflops"], 4))
            gemm_ms += ms
            gemm_flops += amount
        else:
            ach = amount / (ms * 1e-3) / 1e9
            kernels[name] = dict(ms=round(ms, 4), bound="hbm", achieved=round(ach, 1), unit="GB/s",
                                 frac=round(ach / peaks["hbm_gbs"], 4))
    return kernels, gemm_ms, gemm_flops, {n: sum(v) / len(v) for n, v in acc.items()}


def single_gpu_layer_run(cfg, dev, steps, warmup, peaks, seed):
    """One GPU, one MoE layer of shape `cfg`, inputs resident: device-timed ms/step through b200_moe_block_fwd / _bwd
    and the per-op roofline. Used for the target shape beside the headline and as the same-batch base of the
    multi-GPU lines. Frees what it allocated."""
    import torch

    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.moe_layer import MoELayer

    T, d, E, k, f = cfg["T"], cfg["d"], cfg["E"], cfg["k"], cfg["f"]
    gen = torch.Generator(device=dev).manual_seed(seed)

    def normal(shape, std):
        return (torch.randn(shape, generator=gen, device=dev) * std).to(torch.bfloat16)

    X, dOut, Wr = normal((T, d), 1.0), normal((T, d), 1.0), normal((E, d), 0.02)
    W1, W3, W2 = normal((E, f, d), 0.02), normal((E, f, d), 0.02), normal((E, d, f), 0.02)
    out, dXn, dWr = torch.zeros_like(X), torch.empty_like(X), torch.zeros_like(Wr)
    dW1, dW3, dW2 = torch.zeros_like(W1), torch.zeros_like(W3), torch.zeros_like(W2)
    layer = MoELayer(T, d, E, k, f, device=dev)
    block = layer.block(Wr, W1, W3, W2)

    def step():
        out.zero_()
        if layer.profile is None:
            ops.moe_block_fwd(block, X, out)
            ops.moe_block_bwd(block, X, dOut, dXn, dWr, dW1, dW3, dW2)
        else:
            layer.forward(X, Wr, W1, W3, W2, out)
            layer.backward(X, Wr, W1, W3, W2, dOut, dXn, dWr, dW1, dW3, dW2)

    for _ in range(max(3, warmup)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if ops.gemm_status() != 0:
        raise RuntimeError("a GEMM kernel gave up waiting; the timing is void")
    kernels, gemm_ms, gemm_flops, _ = per_op_profile(layer, step, algorithmic_work(cfg), peaks, 3)
    ach = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms else 0.0
    rec = dict(workload=workload_name(cfg, 1), ms_per_step=round(ms, 4), value=T / (ms * 1e-3), unit=UNIT, steps=steps,
               gemm_tflops=round(ach, 1), gemm_frac_of_sustained_peak=round(ach / peaks["bf16_tflops_sustained"], 4),
               gemm_frac_of_burst_peak=round(ach / peaks["bf16_tflops"], 4), gemm_ms_per_step=round(gemm_ms, 4))
    del layer, block, X, dOut, Wr, W1, W3, W2, out, dXn, dWr, dW1, dW3, dW2
    torch.cuda.empty_cache()
    return rec


def run_gpu_arm(args, world):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        import datetime

        # a bounded collective timeout: a rank that falls out of step ends the run in minutes, not in ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=300))
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.moe_layer import MoELayer

    cfg = dict(CFG_1GPU if world == 1 else CFG_EP)
    if args.tokens > 0:
        cfg["T"] = args.tokens
    T, d, E, k, f = cfg["T"], cfg["d"], cfg["E"], cfg["k"], cfg["f"]
    steps, warmup = max(1, args.steps), (max(0, args.warmup) if args.quick else max(3, args.warmup))
    peaks = read_peaks()
    dev = torch.device("cuda", local_rank)
    gen = torch.Generator(device=dev).manual_seed(0xB200 + rank)

    def normal(shape, std):
        return (torch.randn(shape, generator=gen, device=dev) * std).to(torch.bfloat16)

    X, dOut = normal((T, d), 1.0), normal((T, d), 1.0)
    wgen = torch.Generator(device=dev).manual_seed(0xB2000003)  # router weight identical on every rank
    Wr = (torch.randn((E, d), generator=wgen, device=dev) * 0.02).to(torch.bfloat16)

    transport = None
    if world == 1:
        layer = MoELayer(T, d, E, k, f, device=dev)
        E_loc = E
    else:
        from ml_dataflow_b200.ep import ExpertParallelMoELayer

        # "fused" (default): rows out through the gather kernel, back through the epilogue of the last GEMM of each
        # pass, driven op by op from ep.py. "c": the same buffers and kernels driven by b200_ep_moe_block_fwd / _bwd, one C
        # call per direction with the library's own barrier / plan kernels; it is also timed after the main region
        # (`c_driver`). The two measure within about 3 % of each other at 2, 4 and 8 GPUs.
        transport = os.environ.get("B200_EP_TRANSPORT", "fused")
        layer = ExpertParallelMoELayer(T, d, E, k, f, dist, device=dev, transport="fused" if transport == "c" else transport,
                                       slices=int(os.environ.get("B200_EP_SLICES", "1")))
        E_loc = E // world
    W1, W3, W2 = normal((E_loc, f, d), 0.02), normal((E_loc, f, d), 0.02), normal((E_loc, d, f), 0.02)
    out = torch.zeros((T, d), dtype=torch.bfloat16, device=dev)
    dXn = torch.empty_like(out)
    dWr = torch.zeros_like(Wr)
    dW1, dW3, dW2 = torch.zeros_like(W1), torch.zeros_like(W3), torch.zeros_like(W2)

    exchange_note = None
    block = layer.block(Wr, W1, W3, W2) if world == 1 else None
    ep_block = layer.c_block(Wr, W1, W3, W2) if transport == "c" else None

    def step(Xs, dOs, outs, dXs):
        outs.zero_()
        if block is not None and layer.profile is None:
            # one C call per direction (b200_moe_block_fwd / _bwd): the call a C host makes
            ops.moe_block_fwd(block, Xs, outs)
            ops.moe_block_bwd(block, Xs, dOs, dXs, dWr, dW1, dW3, dW2)
        elif ep_block is not None and layer.profile is None:
            ops.ep_moe_block_fwd(ep_block, Xs, outs)
            ops.ep_moe_block_bwd(ep_block, Xs, dOs, dXs, dWr, dW1, dW3, dW2)
        else:
            # the same op sequence issued from Python, with events between the ops when profiling
            layer.forward(Xs, Wr, W1, W3, W2, outs)
            layer.backward(Xs, Wr, W1, W3, W2, dOs, dXs, dWr, dW1, dW3, dW2)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------- device-resident timing
    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.quick:
        sampler.start()
    t_w = time.perf_counter()
    for _ in range(warmup):
        step(X, dOut, out, dXn)
    barrier()
    if ep_block is not None:
        # the C driver's barrier kernels give up after 2 s instead of hanging; if one did during warm-up on any rank,
        # the Python driver of the same kernels (NCCL barriers) takes over and the line says so
        bad = torch.tensor([ops.ep_status()], dtype=torch.int32, device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()) != 0:
            ep_block = None
            transport = "fused"
            exchange_note = "the C driver's barrier timed out in warm-up; timed with the Python driver"
            for _ in range(warmup):
                step(X, dOut, out, dXn)
            barrier()
    if not args.quick:
        # keep the GPUs busy until nvidia-smi has started sampling, so the clock record covers the timed region;
        # every rank runs the same number of extra steps (the step contains collectives when world > 1)
        per_step_ms = max_over_ranks((time.perf_counter() - t_w) * 1e3 / max(1, warmup))
        for _ in range(int(min(60, max(1, 1200.0 / max(per_step_ms, 1.0))))):
            step(X, dOut, out, dXn)
        barrier()
    ops.LAUNCHES = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        step(X, dOut, out, dXn)
    e1.record()
    barrier()
    launches = ops.LAUNCHES
    ms_step = max_over_ranks(e0.elapsed_time(e1) / steps)
    clocks = sampler.stop() if rank == 0 else None
    status = ops.gemm_status()
    if status != 0:
        raise RuntimeError(f"a GEMM kernel gave up waiting (status {status}); the timing is void")
    if world > 1:
        layer.check()  # raises if a receive buffer overflowed (rows dropped): the timing would be void
    value = world * T / (ms_step * 1e-3)
    if args.quick:
        if rank == 0:
            print(json.dumps(dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=steps, warmup=warmup,
                                  ms_per_step=ms_step, quick=True, gpu_launches=launches,
                                  config=dict(workload=workload_name(cfg, world)))), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---------------- end to end: pinned host buffers, copies inside the timed region, double buffered
    # The pinned buffers are first touched while this process is confined to the CPUs of the GPU's own NUMA node, so
    # that the pages sit on the memory that node's PCIe root reaches directly (eight ranks that all pin on one node
    # share one memory controller and the inter-socket link).
    numa_node, numa_cpus = gpu_numa_cpus(local_rank)
    old_aff = None
    if numa_cpus and hasattr(os, "sched_setaffinity"):
        try:
            old_aff = os.sched_getaffinity(0)
            os.sched_setaffinity(0, numa_cpus & old_aff or old_aff)
        except OSError:
            old_aff = None

    def pinned_like(t):
        return torch.empty(t.shape, dtype=t.dtype).pin_memory()

    Xh, dOh = pinned_like(X), pinned_like(dOut)
    Xh.copy_(X)
    dOh.copy_(dOut)
    outh = [pinned_like(X).zero_() for _ in range(2)]
    dXh = [pinned_like(X).zero_() for _ in range(2)]
    if old_aff is not None:
        os.sched_setaffinity(0, old_aff)
    Xd, dOd = [torch.empty_like(X) for _ in range(2)], [torch.empty_like(X) for _ in range(2)]
    outd, dXd = [torch.empty_like(X) for _ in range(2)], [torch.empty_like(X) for _ in range(2)]
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_loop(n):
        with torch.cuda.stream(s_in):
            Xd[0].copy_(Xh, non_blocking=True)
            dOd[0].copy_(dOh, non_blocking=True)
            ev_in[0].record(s_in)
        for i in range(n):
            c, nx = i % 2, (i + 1) % 2
            if i + 1 < n:
                with torch.cuda.stream(s_in):
                    if i >= 1:
                        s_in.wait_event(ev_comp[nx])  # step i-1 has finished reading buffer nx
                    Xd[nx].copy_(Xh, non_blocking=True)
                    dOd[nx].copy_(dOh, non_blocking=True)
                    ev_in[nx].record(s_in)
            main.wait_event(ev_in[c])
            if i >= 2:
                main.wait_event(ev_out[c])  # results of step i-2 have left buffer c
            step(Xd[c], dOd[c], outd[c], dXd[c])
            ev_comp[c].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[c])
                outh[c].copy_(outd[c], non_blocking=True)
                dXh[c].copy_(dXd[c], non_blocking=True)
                ev_out[c].record(s_out)
        main.wait_event(ev_out[0])
        main.wait_event(ev_out[1])

    e2e_loop(2)
    barrier()
    e0.record()
    e2e_loop(steps)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / steps)
    e2e_value = world * T / (ms_e2e * 1e-3)
    io_bytes = 2 * T * d * 2

    # host link alone: the step's H2D and D2H copies with nothing else running, every rank at once (what the host
    # path delivers per GPU when all N share it)
    def copies_only(n):
        for _ in range(n):
            with torch.cuda.stream(s_in):
                Xd[0].copy_(Xh, non_blocking=True)
                dOd[0].copy_(dOh, non_blocking=True)
            with torch.cuda.stream(s_out):
                outh[0].copy_(outd[0], non_blocking=True)
                dXh[0].copy_(dXd[0], non_blocking=True)

    copies_only(1)
    barrier()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0.record(s_in)
    o0.record(s_out)
    copies_only(4)
    h1.record(s_in)
    o1.record(s_out)
    barrier()
    h2d_gbs = 4 * io_bytes / (h0.elapsed_time(h1) * 1e-3) / 1e9
    d2h_gbs = 4 * io_bytes / (o0.elapsed_time(o1) * 1e-3) / 1e9
    if dist is not None:
        tmin = torch.tensor([h2d_gbs, d2h_gbs], dtype=torch.float64, device=dev)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
        h2d_gbs, d2h_gbs = float(tmin[0]), float(tmin[1])
    del Xd, dOd, outd, dXd, Xh, dOh, outh, dXh

    # ---------------- per-op timing for the roofline (separate pass, events between ops)
    kernels, gemm_ms, gemm_flops, raw_ms = per_op_profile(layer, lambda: step(X, dOut, out, dXn), algorithmic_work(cfg),
                                                          peaks, max(3, min(steps, 10)))
    if world > 1:
        link = NVLINK_PEER_GBS_RECORDED
        for name, amount in exchange_work(cfg, world).items():
            if name in raw_ms:
                ms = raw_ms[name]
                if transport in ("fused", "c") and name.startswith("return"):
                    # the rows went home inside the GEMM epilogues; what is left of this phase is the barrier
                    kernels[name] = dict(ms=round(ms, 4), bound="barrier (rows are stored by the GEMM epilogue)")
                    continue
                ach_x = amount / (ms * 1e-3) / 1e9
                kernels[name] = dict(ms=round(ms, 4), bound="nvlink", achieved=round(ach_x, 1), unit="GB/s per direction",
                                     peak=round(link, 1), frac=round(ach_x / link, 4),
                                     peak_source="recorded peer-copy rate per direction for this machine type (nominal "
                                                 "900 GB/s); a constant, not measured by this run")
    ach = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms else 0.0
    traffic = NCU_GEMM_DRAM_BYTES_PER_STEP.get((T, d, E, k, f)) if world == 1 else None
    roofline = dict(kernel="gemm_sm100_kernel (grouped expert GEMMs: 7 launches per step, 18*R*d*f flop)",
                    bound="tensor", achieved=round(ach, 1), peak=peaks["bf16_tflops_sustained"], unit="TFLOP/s",
                    frac=round(ach / peaks["bf16_tflops_sustained"], 4),
                    frac_of_burst_peak=round(ach / peaks["bf16_tflops"], 4), peak_source=peaks["source"] +
                    " (sustained cuBLAS bf16, the kernel is timed inside a long step)",
                    traffic=traffic, traffic_unit="bytes per step over the 7 launches",
                    traffic_source=NCU_TRAFFIC_SOURCE if traffic else None, algorithmic_flop=gemm_flops,
                    ms_per_step_in_kernel=round(gemm_ms, 4))

    # ---------------- after the timed regions: the target shape / the same-batch base on one GPU, EP parity
    extra = {}
    if world > 1 and transport == "fused":
        # the C driver of the same buffers and kernels, a short device-timed loop (every rank takes the same path: the
        # status votes are reduced over the ranks before anything depends on them)
        try:
            ep_c = layer.c_block(Wr, W1, W3, W2)

            def step_c():
                out.zero_()
                ops.ep_moe_block_fwd(ep_c, X, out)
                ops.ep_moe_block_bwd(ep_c, X, dOut, dXn, dWr, dW1, dW3, dW2)

            for _ in range(3):
                step_c()
            barrier()
            bad_c = torch.tensor([1 if ops.ep_status() != 0 else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(bad_c, op=dist.ReduceOp.MAX)
            if int(bad_c.item()) != 0:
                extra["c_driver"] = dict(error="a barrier of the C driver timed out")
            else:
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                barrier()
                c0.record()
                for _ in range(5):
                    step_c()
                c1.record()
                barrier()
                ms_c = max_over_ranks(c0.elapsed_time(c1) / 5)
                layer.check()
                extra["c_driver"] = dict(ms_per_step=round(ms_c, 3), value=round(world * T / (ms_c * 1e-3), 1), unit=UNIT, steps=5,
                                         note="b200_ep_moe_block_fwd / _bwd: one C call per direction, device barriers")
        except Exception as exc:  # the main line stands without it
            extra["c_driver"] = dict(error=f"{type(exc).__name__}: {str(exc)[:200]}")
    del layer, block, ep_block
    torch.cuda.empty_cache()
    if world == 1 and args.tokens <= 0:
        # the target shape (T=32768 on one GPU) beside the headline configuration
        extra["ns_shape"] = single_gpu_layer_run(CFG_NS, dev, 10, 3, peaks, 0xB200)
        torch.cuda.empty_cache()
        extra["block_ops"] = block_ops_profile(dev, peaks)
        torch.cuda.empty_cache()
        try:
            extra["decoder_step"] = decoder_step_run(dev, peaks)
        except Exception as exc:  # the headline line does not depend on it
            extra["decoder_step"] = dict(error=f"{type(exc).__name__}: {str(exc)[:200]}")
    if world > 1:
        ep_parity = "ok"
        try:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            from ep_parity import check_expert_parallel

            check_expert_parallel(dist, rank, world, transport, num_experts=max(8, world))
        except Exception as exc:  # reported below, after every rank has voted
            ep_parity = f"rank {rank}: {type(exc).__name__}: {str(exc)[:300]}"
        votes = [None] * world
        dist.all_gather_object(votes, ep_parity)
        bad = [v for v in votes if v != "ok"]
        extra["ep_parity"] = "ok" if not bad else bad[0]
        extra["ep_parity_case"] = (f"{world} ranks, T=384 per rank, d=256, {max(8, world)} experts, top-2, ffn 128, two "
                                   "steps, every rank against the CPU oracle (counts and mappings bit-exact)")
        # the same per-GPU batch on ONE GPU with all 64 experts (no exchange): the base for weak-scaling efficiency
        if rank == 0:
            base = single_gpu_layer_run(dict(cfg), dev, 5, 3, peaks, 0xB200)
            extra["same_batch_1gpu"] = base
            extra["efficiency_same_batch"] = round(value / (world * base["value"]), 4)
        dist.barrier()
        if bad:
            if rank == 0:
                print(json.dumps(dict(metric=METRIC, impl="ours", n_gpus=world, error="expert-parallel parity failed",
                                      ep_parity=bad[0])), flush=True)
            dist.destroy_process_group()
            sys.exit(1)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=steps, warmup=warmup, ms_per_step=ms_step,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic", impl="ours",
                config=dict(workload=workload_name(cfg, world), T=T, d_model=d, experts=E, top_k=k, ffn=f,
                            **({"exchange": transport, "per_op_times_from": "the Python driver of the same kernels (ep.py, events "
                    "between the ops; its barriers are NCCL all-reduces where the C driver uses its own barrier kernel)"
                    if transport == "c" else "the timed driver",
                    **({"exchange_note": exchange_note} if exchange_note else {})} if world > 1 else {}),
                            l2="inputs exceed L2 (zone 2*T*k*d bytes per pass)"),
                e2e=dict(value=e2e_value, unit=UNIT, h2d_bytes_per_step=io_bytes, d2h_bytes_per_step=io_bytes,
                         ms_per_step=ms_e2e, ratio_to_device_timed=round(e2e_value / value, 4),
                         host_link=dict(h2d_gbs_per_gpu=round(h2d_gbs, 2), d2h_gbs_per_gpu=round(d2h_gbs, 2),
                                        note="copies of one step alone, all ranks at once, slowest rank",
                                        needed_gbs_per_gpu=round(io_bytes / (ms_step * 1e-3) / 1e9, 2),
                                        pinned_on_numa_node=numa_node)),
                gpu_launches=launches, clocks=clocks, roofline=roofline, kernels=kernels, **extra)
    if world == 1:
        line["cpu_baseline"], _ = cpu_baseline_record(cfg, 1, 1)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override T (tokens per GPU); for profiler captures")
    ap.add_argument("--quick", action="store_true",
                    help="device-timed loop only, exactly --warmup/--steps iterations (for ncu launch lists)")
    ap.add_argument("--block-ops", action="store_true",
                    help="only the block / head ops record (one GPU; one launch of each kernel per repetition: for ncu)")
    ap.add_argument("--attention", action="store_true", help="with --block-ops: the attention forward / backward too")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    if args.block_ops:
        import torch

        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        print(json.dumps(dict(block_ops=block_ops_profile(dev, read_peaks(), iters=max(1, args.steps if args.steps != 30 else 5),
                                                          with_attention=args.attention))), flush=True)
        return
    if args.impl == "reference":
        run_reference_arm(args, CFG_1GPU if world == 1 else CFG_EP, world)
        return
    if world > 1 and "RANK" not in os.environ:
        sys.exit("for --gpus > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    run_gpu_arm(args, world)


if __name__ == "__main__":
    main()

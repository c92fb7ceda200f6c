"""Benchmark of the compressed-expert MoE layer (one step = one forward pass of one layer).

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference --gpus N --steps K ...  # CPU baseline arm (rank 0 only)

Workload (default ``switch-c-2048``): one Switch-c-2048-shaped sparse layer -- d_model 2080, d_ff
6144, 2048 experts of ternary weights (P(0) = 0.90) compressed with the reference's dictionary
encoder (~4.6 GB), 2048 bf16 tokens ~ N(0,1) routed top-1 by a seeded random router -- expert-parallel
over N GPUs of one node (2048 / N experts and 2048 / N tokens per rank).  Weights are synthetic and
seeded (the Switch checkpoints are not available offline); they are generated and packed on the GPU.

The one JSON line printed by rank 0 carries: ``value`` = tokens/s with inputs resident in HBM (CUDA
events, max over ranks); ``e2e`` = tokens/s with pinned-host inputs and outputs (H2D + layer + D2H in
the timed region); ``roofline`` for the grouped decode-matvec kernel (algorithmic compressed bytes /
event-timed launch duration, against the measured HBM copy bandwidth); ``cpu_baseline`` = the CPU
oracle on a bounded sample of the same experts.
"""
from __future__ import annotations

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

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
SEED = 0
FALLBACK_HBM_GBS = 6650.0

WORKLOADS = {
    # name: (d_model, d_ff, experts, tokens)
    "switch-c-2048": (2080, 6144, 2048, 2048),
    "switch-large-128": (1024, 4096, 128, 512),
    "switch-base-128": (768, 3072, 128, 128),
}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="switch-c-2048", choices=sorted(WORKLOADS))
    p.add_argument("--experts", type=int, default=0, help="override the expert count (debugging)")
    p.add_argument("--tokens", type=int, default=0, help="override the token count (debugging)")
    p.add_argument("--cpu-seconds", type=float, default=12.0, help="target duration of the CPU baseline sample")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA-graph replay")
    p.add_argument("--skew", type=int, default=0,
                   help="skewed router: this many hot experts receive half of the tokens (config 3 uses 8)")
    p.add_argument("--tokens-per-expert", type=int, default=0,
                   help="router override: every expert receives exactly this many tokens (the token count becomes "
                        "experts x this); 1 is the batch-1 case: every matrix is applied to one vector")
    p.add_argument("--no-parity-check", action="store_true", help="skip the oracle check of sampled experts")
    p.add_argument("--no-gpu-reference", action="store_true", help="skip the timing of the reference's own kernel")
    p.add_argument("--min-seconds", type=float, default=1.0,
                   help="the timed loop of --steps steps is repeated until this much time has been timed")
    p.add_argument("--decode-input", default="forced", choices=["forced", "greedy"],
                   help="generate mode: what a decode step is fed (forced: seeded random ids, so that steps visit "
                        "different experts; greedy: the previous step's argmax)")
    p.add_argument("--decode-routing", default="uniform", choices=["uniform", "model"],
                   help="generate mode: uniform = every decode step is sent to a seeded random expert in every block "
                        "(a balanced router); model = the random-init routers decide (a few experts per block)")
    p.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                   help="N > 1: how rows travel between ranks (peer: stored straight into the peers' memory over "
                        "NVLink; nccl: two all-to-all collectives; auto: peer where it can be set up)")
    p.add_argument("--kernel-times", action="store_true",
                   help="also time the kernels of a step (torch profiler, eager launches) and add their average "
                        "durations to the JSON line")
    p.add_argument("--mode", default="moe", choices=["moe", "layers", "generate", "smem-ceiling"],
                   help="moe: the MoE-layer benchmark (default); layers: the reference's per-layer matvec "
                        "benchmark (test.py --benchmark) on its six shapes; generate: end-to-end decoding; "
                        "smem-ceiling: the grouped kernel on weights that stay in L2 (no HBM traffic)")
    return p.parse_args()


def workload_dims(args):
    d_model, d_ff, experts, tokens = WORKLOADS[args.workload]
    experts = args.experts or experts
    tokens = experts * args.tokens_per_expert if args.tokens_per_expert > 0 else (args.tokens or tokens)
    return d_model, d_ff, experts, tokens


def forced_logits(n_tokens, n_experts):
    """Router logits that send token t to expert t % n_experts with probability ~1."""
    import torch
    logits = torch.full((n_tokens, n_experts), -20.0)
    logits[torch.arange(n_tokens), torch.arange(n_tokens) % n_experts] = 20.0
    return logits


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples every 50 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons = [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    out["sm_max_mhz"] = float(f[2])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        out["window"] = "1.5 s of untimed repeats of the step, then the device-timed and the end-to-end region"
        return out


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def recorded_traffic_ratio():
    """DRAM bytes per algorithmic byte of the grouped kernel, from the committed ncu summary."""
    try:
        with open(os.path.join(ROOT, "profiles", "k_matmul_grouped.traffic.json")) as f:
            return float(json.load(f)["dram_bytes_per_algorithmic_byte"])
    except Exception:
        return None


# ---------------------------------------------------------------------------------------------
# CPU baseline (the oracle: C port of the reference's CPU decode + matmul path)
# ---------------------------------------------------------------------------------------------
def cpu_sample_experts(d_model, d_ff, expert_ids):
    """Build the same seeded experts on the CPU (oracle generator + oracle encoder)."""
    import numpy as np
    from oracle import oracle as O
    from qmoe_b200 import synth
    _, trie = O.build_dictionary()
    out = []
    for e in expert_ids:
        mats = []
        for which, (h, w) in enumerate(((d_ff, d_model), (d_model, d_ff))):
            m = 2 * e + which
            sym = O.synth_ternary(h * w, SEED, synth.matrix_first_index(m), 0.9).reshape(h, w)
            codes, row_off = O.encode_matrix(trie, sym)
            mm = synth.row_scales(h, SEED, m)
            mats.append((codes, row_off, mm.view(__import__("torch").int16).numpy().view(np.uint16)))
        out.append(mats)
    return out


def cpu_time_sample(d_model, d_ff, experts, x_bits):
    """Seconds to push one token through each sampled expert with the oracle (all host threads)."""
    from oracle import oracle as O
    dec, _ = O.build_dictionary()
    t0 = time.perf_counter()
    for i, (wi, wo) in enumerate(experts):
        O.expert_ffn(dec, wi, wo, x_bits[i % x_bits.shape[0]:i % x_bits.shape[0] + 1], d_model, d_ff)
    return time.perf_counter() - t0


def cpu_baseline(args, d_model, d_ff, n_experts):
    import numpy as np
    from oracle import oracle as O
    from qmoe_b200 import synth
    O.use_all_cores()
    x = synth.tokens(64, d_model, SEED)
    x_bits = x.view(__import__("torch").int16).numpy().view(np.uint16)
    probe = cpu_sample_experts(d_model, d_ff, [0])
    cpu_time_sample(d_model, d_ff, probe, x_bits)
    per = max(cpu_time_sample(d_model, d_ff, probe, x_bits), 1e-4)
    count = int(max(2, min(n_experts, 256, args.cpu_seconds / per)))
    experts = probe + cpu_sample_experts(d_model, d_ff, list(range(1, count)))
    secs = cpu_time_sample(d_model, d_ff, experts, x_bits)
    return {
        "value": count / secs, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
        "sample": f"{count} experts x 1 token each ({args.workload} shapes), C port of the reference's CPU "
                  f"decode (test.py:103-115) + matmul, OpenMP over rows, {secs:.2f} s",
    }


def run_reference(args):
    """CPU arm: rank 0 alone times the oracle port on bounded samples of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as O
    from qmoe_b200 import synth
    O.build()
    O.use_all_cores()                  # torchrun exports OMP_NUM_THREADS=1
    d_model, d_ff, n_experts, n_tokens = workload_dims(args)
    x = synth.tokens(64, d_model, SEED)
    x_bits = x.view(__import__("torch").int16).numpy().view(np.uint16)
    probe = cpu_sample_experts(d_model, d_ff, [0])
    cpu_time_sample(d_model, d_ff, probe, x_bits)
    per = max(cpu_time_sample(d_model, d_ff, probe, x_bits), 1e-4)
    budget = 90.0 / max(args.steps + args.warmup, 1)           # whole run within a few minutes
    count = int(max(2, min(n_experts, 64, budget / per)))
    experts = probe + cpu_sample_experts(d_model, d_ff, list(range(1, count)))
    for _ in range(args.warmup):
        cpu_time_sample(d_model, d_ff, experts, x_bits)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_time_sample(d_model, d_ff, experts, x_bits)
    value = count * args.steps / t
    sample = (f"{count} experts x 1 token per step ({args.workload} shapes); C port of the reference's CPU "
              f"decode (test.py:103-115) + matmul; OpenMP over rows")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded ternary experts, P(0)=0.90)",
        "config": {"workload": args.workload, "d_model": d_model, "d_ff": d_ff, "experts": n_experts,
                   "tokens": n_tokens, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# this implementation
# ---------------------------------------------------------------------------------------------
def parity_leg(world, rank, dev, out, index, prob, hidden_all, d_model, d_ff, e_local):
    """After the timed regions: outputs of the tokens of a few of rank 0's experts against the CPU
    oracle (the experts are regenerated from the seed and encoded by the oracle's own encoder).
    ``out`` / ``index`` / ``prob``: this rank's layer output, expert choice and router probability."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    if world > 1:
        outs = [torch.empty_like(out) for _ in range(world)]
        idxs = [torch.empty_like(index) for _ in range(world)]
        prbs = [torch.empty_like(prob) for _ in range(world)]
        dist.all_gather(outs, out.contiguous())
        dist.all_gather(idxs, index.contiguous())
        dist.all_gather(prbs, prob.contiguous())
        out, index, prob = torch.cat(outs), torch.cat(idxs), torch.cat(prbs)
    if rank != 0:
        return None
    out, index, prob = out.float().cpu(), index.cpu().long(), prob.float().cpu()
    counts = torch.bincount(index, minlength=e_local)[:e_local]
    order = torch.argsort(counts, descending=True).tolist()
    chosen = order[:1] + [e for e in order if counts[e] == 2][:1] + [e for e in order if counts[e] == 1][:2]
    chosen = [e for e in dict.fromkeys(chosen) if counts[e] > 0]
    O.use_all_cores()
    dec, _ = O.build_dictionary()
    worst, n_tok = 0.0, 0
    for e in chosen:
        wi, wo = cpu_sample_experts(d_model, d_ff, [e])[0]
        tok = torch.nonzero(index == e).reshape(-1)
        x_bits = hidden_all[tok].contiguous().view(torch.int16).numpy().view(np.uint16)
        y = O.expert_ffn(dec, wi, wo, x_bits, d_model, d_ff)
        ref = torch.from_numpy(y.view(np.int16)).view(torch.bfloat16).float() * prob[tok].unsqueeze(1)
        ref = ref.bfloat16().float()
        err = float((out[tok] - ref).abs().max() / max(float(ref.abs().max()), 1e-12))
        worst = max(worst, err)
        n_tok += len(tok)
    return {"experts": chosen, "tokens": n_tok, "max_rel_err": worst, "tolerance": 1e-2,
            "against": "CPU oracle (decode-then-matmul FFN, fp32 accumulation, bf16 hidden activation) x router "
                       "probability; error = max|out - ref| / max|ref| per expert"}


def gpu_reference_leg(store, dev, d_model, d_ff, counts, hidden_dev, ours_tokens_per_s):
    """The reference's own kernel (built unmodified into oracle/_ref), driven as the reference drives
    it -- per active expert, per token, zero y, sub1matvec, ReLU, sub1matvec (sub1.py:139-142,315-317)
    -- on a bounded sample of this rank's experts."""
    import torch
    from qmoe_b200 import sub1
    if (d_ff, d_model) not in LAYER_SHAPES or (d_model, d_ff) not in LAYER_SHAPES:
        return {"unavailable": "the reference kernel handles its six hard-coded shapes only (sub1_cuda_kernel.cu:82-87)"}
    if store.codes is None:
        return {"unavailable": "the store dropped its row-by-row streams"}
    try:
        from oracle import build_ref
        ref = build_ref.load()
    except Exception as exc:
        return {"unavailable": f"oracle/_ref could not be loaded: {exc}"}
    if ref is None:
        return {"unavailable": "oracle/_ref not built (python oracle/build_ref.py, needs the reference checkout)"}
    dec = sub1.DEC(dev)
    sample = [(e, c) for e, c in enumerate(counts) if c > 0][:16]
    mats = [[tuple(t.contiguous() for t in store.matrix(2 * e + w)) for w in (0, 1)] for e, _ in sample]
    n_tok = sum(c for _, c in sample)

    def run():
        pos = 0
        for (e, c), (wi, wo) in zip(sample, mats):
            x = hidden_dev[pos:pos + c]
            h = torch.zeros((c, d_ff), dtype=torch.bfloat16, device=dev)
            for i in range(c):
                ref.sub1matvec(dec, wi[0], wi[1], wi[2], x[i], h[i])
            h = torch.relu(h)
            y = torch.zeros((c, d_model), dtype=torch.bfloat16, device=dev)
            for i in range(c):
                ref.sub1matvec(dec, wo[0], wo[1], wo[2], h[i], y[i])
            pos += c

    for _ in range(3):
        run()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    reps = 0
    t0 = time.perf_counter()
    a.record()
    while reps < 200 and (reps < 5 or time.perf_counter() - t0 < 0.5):
        run()
        reps += 1
    b.record()
    torch.cuda.synchronize()
    value = n_tok * reps / (a.elapsed_time(b) * 1e-3)
    return {"value": value, "unit": UNIT, "kind": "the reference's CUDA kernel, unmodified, built for sm_100",
            "sample": f"{len(sample)} active experts of this layer with their {n_tok} routed tokens, {reps} repeats; one "
                      "sub1matvec launch per token and linear plus torch zeros / relu, CUDA events, no host "
                      "synchronisation between calls; every expert costs the same, so tokens/s of the sample is "
                      "tokens/s of the layer",
            "ours_over_reference": ours_tokens_per_s / value if value > 0 else None}


def l2_resident_rate(dev, d_model, d_ff, n_experts, hidden, logits, lib):
    """The benchmark's own step -- same tokens, same routing, same work list -- over weights that stay
    in L2: a layer whose `n_experts` experts alias the matrices of EIGHT real experts (19 MB of code
    streams in a 126 MB L2).  After the first pass no grouped launch reads codes from HBM, so the rate
    is what the SMs' issue and shared-memory pipes sustain for this decoder on this workload with the
    memory system out of the picture.  Returns the milliseconds of the grouped launches per step."""
    import ctypes
    import torch
    from qmoe_b200 import _lib, sub1, synth
    real = 8
    base = synth.build_store(d_model, d_ff, list(range(real)), SEED, dev)
    layer = sub1.FasterMLP(None, base.aliased(n_experts), expert_capacity=1024)
    h, lg = hidden.unsqueeze(0), logits.unsqueeze(0)
    for _ in range(3):
        layer(h, router_logits=lg)
    lib.qmoe_profile_enable(1)
    for _ in range(10):
        layer(h, router_logits=lg)
    torch.cuda.synchronize()
    lib.qmoe_profile_enable(0)
    wi_ms, wo_ms, calls = ctypes.c_float(), ctypes.c_float(), ctypes.c_int()
    _lib.check(lib.qmoe_profile_read(ctypes.byref(wi_ms), ctypes.byref(wo_ms), ctypes.byref(calls)))
    return (wi_ms.value + wo_ms.value) / max(calls.value, 1), real


def run_smem_ceiling(args):
    """Only the on-chip ceiling: the workload's step (seeded uniform routing) timed over the real layer
    in HBM and over the same layer with its experts aliased onto eight real ones, which stay in L2.
    One JSON line; single GPU."""
    import ctypes
    import torch
    from qmoe_b200 import _lib, sub1, synth
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path for the sub1 kernels")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _lib.load()
    d_model, d_ff, n_experts, n_tokens = workload_dims(args)
    store = synth.build_store(d_model, d_ff, list(range(n_experts)), SEED, dev)
    hidden = synth.tokens(n_tokens, d_model, SEED + 1).to(dev)
    logits = (forced_logits(n_tokens, n_experts) if args.tokens_per_expert > 0
              else synth.router_logits(n_tokens, n_experts, SEED + 2)).to(dev)
    layer = sub1.FasterMLP(None, store, expert_capacity=1024)
    h, lg = hidden.unsqueeze(0), logits.unsqueeze(0)
    for _ in range(max(args.warmup, 3)):
        _, (_, index) = layer(h, router_logits=lg)
    lib.qmoe_profile_enable(1)
    for _ in range(max(args.steps, 1)):
        layer(h, router_logits=lg)
    torch.cuda.synchronize()
    lib.qmoe_profile_enable(0)
    wi_ms, wo_ms, calls = ctypes.c_float(), ctypes.c_float(), ctypes.c_int()
    _lib.check(lib.qmoe_profile_read(ctypes.byref(wi_ms), ctypes.byref(wo_ms), ctypes.byref(calls)))
    ms_hbm = (wi_ms.value + wo_ms.value) / max(calls.value, 1)
    counts = torch.bincount(index.reshape(-1).long(), minlength=n_experts).cpu().tolist()
    alg = sum(store.matrix_bytes(2 * e) + store.matrix_bytes(2 * e + 1) + 4 * c * (d_model + d_ff)
              for e, c in enumerate(counts) if c > 0)
    codes = sum(store.host_descs[2 * e].n_codes + store.host_descs[2 * e + 1].n_codes for e, c in enumerate(counts) if c > 0)
    del layer, store
    torch.cuda.empty_cache()
    ms_l2, real = l2_resident_rate(dev, d_model, d_ff, n_experts, hidden, logits, lib)
    peak, peak_kind = measured_hbm_peak()
    sm_hz = 1965.0e6
    print(json.dumps({
        "mode": "smem-ceiling", "config": {"workload": args.workload, "experts": n_experts, "tokens": n_tokens},
        "grouped_ms_per_step_hbm_resident": ms_hbm, "grouped_ms_per_step_l2_resident": ms_l2,
        "frac_of_on_chip_ceiling": ms_l2 / ms_hbm if ms_hbm > 0 else None,
        "algorithmic_bytes_per_step": alg,
        "achieved_gbs": alg / (ms_hbm * 1e-3) / 1e9, "ceiling_gbs": alg / (ms_l2 * 1e-3) / 1e9,
        "hbm_peak_gbs": peak, "hbm_peak_kind": peak_kind,
        "codes_per_sm_per_clock_hbm_resident": codes / (ms_hbm * 1e-3) / (148 * sm_hz),
        "codes_per_sm_per_clock_at_ceiling": codes / (ms_l2 * 1e-3) / (148 * sm_hz),
        "what": f"ceiling = the same step (same tokens, routing, work list) on a layer whose {n_experts} experts "
                f"alias the matrices of {real} real experts, so every code stream stays in L2: what the SMs' issue and "
                "shared-memory pipes sustain for this decoder with the memory system out of the picture"}), flush=True)


def run_ours(args):
    import ctypes
    import torch
    import torch.distributed as dist
    from qmoe_b200 import _lib, sub1, synth
    from qmoe_b200.ep import ExpertParallelMLP, default_pair_capacity

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path for the sub1 kernels")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    d_model, d_ff, n_experts, n_tokens = workload_dims(args)
    assert n_experts % world == 0 and n_tokens % world == 0
    e_local, t_local = n_experts // world, n_tokens // world
    lib = _lib.load()

    t_setup = time.perf_counter()
    store = synth.build_store(d_model, d_ff, list(range(rank * e_local, (rank + 1) * e_local)), SEED, dev)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    g = torch.Generator().manual_seed(SEED * 31 + 5)
    router_weight = (torch.randn(n_experts, d_model, generator=g) / d_model ** 0.5).bfloat16().float()
    hidden_all = synth.tokens(n_tokens, d_model, SEED)
    hidden_host = hidden_all[rank * t_local:(rank + 1) * t_local].contiguous().pin_memory()
    out_host = torch.empty_like(hidden_host).pin_memory()
    hidden_dev = hidden_host.to(dev)
    # router logits given directly (skewed router, or exactly k tokens per expert); otherwise the
    # layer's own classifier computes them from the hidden states
    given_all = None
    if args.tokens_per_expert > 0:
        given_all = forced_logits(n_tokens, n_experts)
        router = f"every expert receives exactly {args.tokens_per_expert} token(s)"
    elif args.skew > 0:   # N(0,1) plus a large bias that sends half the tokens to the hot experts
        given_all = synth.router_logits(n_tokens, n_experts, SEED, hot_experts=args.skew, hot_fraction=0.5)
        perm = torch.randperm(n_tokens, generator=torch.Generator().manual_seed(SEED))
        given_all = given_all[perm].contiguous()                # spread the hot tokens over the ranks
        router = f"skewed: {args.skew} experts get half of the tokens"
    else:
        router = "uniform top-1"
    given = None if given_all is None else given_all[rank * t_local:(rank + 1) * t_local].contiguous().to(dev)
    if world > 1:
        layer = ExpertParallelMLP(router_weight, store, n_experts, expert_capacity=1024, exchange=args.exchange)
        full = lambda h, lg: layer(h, router_logits=lg, seq_len=t_local)  # noqa: E731
    else:
        layer = sub1.FasterMLP(router_weight, store, expert_capacity=1024)

        def full(h, lg):
            o, (rl, ix) = layer(h.unsqueeze(0), router_logits=None if lg is None else lg.unsqueeze(0))
            return o.squeeze(0), (rl.squeeze(0), ix.squeeze(0))
    step = lambda h: full(h, given)[0]  # noqa: E731

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, finish=None):
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()                       # the timing stream waits for copies on other streams
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def timed_repeats(fn, steps, finish=None):
        """The loop of `steps` steps, repeated until args.min_seconds have been timed (rank 0
        decides, every rank runs the same repeats); returns the per-repeat milliseconds."""
        out, total = [], 0.0
        go = torch.ones(1, device=dev)
        while float(go.item()) > 0:
            ms = timed(fn, steps, finish)
            out.append(ms)
            total += ms
            go.fill_(1.0 if (total < args.min_seconds * 1e3 and len(out) < 200) else 0.0)
            if world > 1:
                dist.broadcast(go, 0)
        return out

    # warm-up (also builds the per-device sparse table and sizes the allocator's pools)
    for _ in range(max(args.warmup, 3)):
        step(hidden_dev)
    barrier()

    # eager pass: kernel durations (CUDA events around the grouped launches of wi and of wo, on their
    # stream) and the launch count; the same kernels are then replayed from a CUDA graph for the
    # headline number
    launches0 = lib.qmoe_launch_count()
    lib.qmoe_profile_enable(1)
    ms_eager = timed(lambda: step(hidden_dev), args.steps)
    lib.qmoe_profile_enable(0)
    launches = (lib.qmoe_launch_count() - launches0) // max(args.steps, 1)
    wi_ms, wo_ms, n_calls = ctypes.c_float(), ctypes.c_float(), ctypes.c_int()
    _lib.check(lib.qmoe_profile_read(ctypes.byref(wi_ms), ctypes.byref(wo_ms), ctypes.byref(n_calls)))

    gstep = None
    if not args.no_graph:
        from qmoe_b200.graph import GraphedStep
        ok = torch.ones(1, device=dev)
        try:
            gstep = GraphedStep(step, hidden_dev)
        except Exception as exc:  # capture unsupported: keep the eager path on every rank
            sys.stderr.write(f"[bench] CUDA-graph capture failed on rank {rank}: {exc}\n")
            ok.zero_()
            gstep = None
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            gstep = None
    run = (lambda: gstep.replay()) if gstep is not None else (lambda: step(hidden_dev))
    for _ in range(3):
        run()
    barrier()

    # nvidia-smi needs most of a second before its first sample and a step can be under a
    # millisecond, so the sampler starts here and the step is repeated, untimed, until it has had
    # 1.5 s under load; the timed regions follow directly.  Every rank runs the same repeats (the
    # step contains collectives), rank 0 decides when to stop.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_load = time.perf_counter()
    go = torch.ones(1, device=dev)
    while float(go.item()) > 0:
        for _ in range(20):
            run()
        torch.cuda.synchronize()
        go.fill_(1.0 if time.perf_counter() - t_load < 1.5 else 0.0)
        if world > 1:
            dist.broadcast(go, 0)
    barrier()
    reps = timed_repeats(run, args.steps)
    ms_sorted = sorted(reps)
    ms_total = ms_sorted[len(ms_sorted) // 2]               # the median repeat is the reported one

    # end to end: pinned host input -> device -> layer -> pinned host output, every step.  With the
    # step in a graph the copies of neighbouring steps overlap its execution (PipelinedStep).
    from qmoe_b200.graph import PipelinedStep
    pipe = PipelinedStep(gstep) if gstep is not None else None

    def e2e_step():
        if pipe is not None:
            pipe.submit(hidden_host, out_host)
        else:
            hidden_dev.copy_(hidden_host, non_blocking=True)
            out_host.copy_(step(hidden_dev), non_blocking=True)

    finish = pipe.drain if pipe is not None else None
    for _ in range(3):
        e2e_step()
    if finish is not None:
        finish()
    e2e_reps = sorted(timed_repeats(e2e_step, args.steps, finish))
    ms_e2e = e2e_reps[len(e2e_reps) // 2]
    clocks = sampler.stop() if rank == 0 else None

    # status words of the timed steps: tile kernels that gave up, tokens that did not fit the exchange
    tile_timeouts = sub1.tile_timeouts(dev, reset=True)
    overflow = layer.overflow_count(reset=True) if world > 1 else 0
    peer_timeouts = layer.peer_timeouts() if world > 1 else 0
    status = torch.tensor([tile_timeouts, overflow, peer_timeouts], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.SUM)
    tile_timeouts, overflow, peer_timeouts = (int(v) for v in status.tolist())

    # one more eager step whose output is checked: expert choice, router probability, layer output
    out_chk, (rl_chk, index_chk) = full(hidden_dev, given)
    _, prob_chk = sub1.route_top1(rl_chk.reshape(t_local, n_experts).float().contiguous())
    parity = None
    if not args.no_parity_check:
        parity = parity_leg(world, rank, dev, out_chk, index_chk.reshape(-1).to(torch.int32), prob_chk, hidden_all,
                            d_model, d_ff, e_local)

    kernel_times = None
    if args.kernel_times:
        # five eager steps under the torch profiler (CUPTI) on every rank; rank 0 reports its own
        from torch.profiler import ProfilerActivity, profile
        barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(5):
                step(hidden_dev)
            torch.cuda.synchronize()
        barrier()
        rows = [e for e in prof.key_averages() if e.device_type == torch.autograd.DeviceType.CUDA]
        total = sum(e.device_time_total for e in rows)
        kernel_times = {
            "per_step_us": round(total / 5, 1), "launches_per_step": sum(e.count for e in rows) / 5,
            "kernels": [{"name": e.key[:70], "calls_per_step": e.count / 5,
                         "avg_us": round(e.device_time_total / max(e.count, 1), 2),
                         "share": round(e.device_time_total / max(total, 1e-9), 4)}
                        for e in sorted(rows, key=lambda e: -e.device_time_total)[:24]]}

    # algorithmic bytes of the grouped kernels on rank 0: matrices of experts that received tokens
    idx_all = index_chk.reshape(-1).to(torch.int64)
    if world > 1:
        parts = [torch.empty_like(idx_all) for _ in range(world)]
        dist.all_gather(parts, idx_all.contiguous())
        idx_all = torch.cat(parts)
    counts = torch.bincount(idx_all, minlength=n_experts)[rank * e_local:(rank + 1) * e_local].cpu().tolist()
    bytes_wi = bytes_wo = 0
    active = 0
    for e, c in enumerate(counts):
        if c > 0:
            active += 1
            bytes_wi += store.matrix_bytes(2 * e) + 2 * c * (d_model + d_ff)
            bytes_wo += store.matrix_bytes(2 * e + 1) + 2 * c * (d_model + d_ff)

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        calls = max(n_calls.value, 1)
        # one persistent launch runs the items of both linears (or, with the fusion switched off, two
        # launches whose average is reported)
        # (the library reports one duration for the fused launch and next to nothing for the second linear)
        fused = wo_ms.value < 0.02 * wi_ms.value
        per_step = 1 if fused else 2
        kernel_ms = (wi_ms.value + wo_ms.value) / (per_step * calls)
        alg_bytes = (bytes_wi + bytes_wo) / per_step                   # algorithmic bytes per launch
        achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9 if kernel_ms > 0 else 0.0
        ratio = recorded_traffic_ratio()
        value = n_tokens * args.steps / (ms_total * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded ternary experts P(0)=0.90 packed by the GPU encoder; N(0,1) tokens; random router)",
            "ms_per_step_repeats": {"repeats": len(reps), "median": ms_total / args.steps,
                                    "min": ms_sorted[0] / args.steps, "max": ms_sorted[-1] / args.steps,
                                    "timed_seconds": sum(reps) * 1e-3,
                                    "note": f"the loop of {args.steps} steps repeated until {args.min_seconds} s were "
                                            "timed; value and ms_per_step are the median repeat"},
            "config": {
                "workload": args.workload, "d_model": d_model, "d_ff": d_ff, "experts": n_experts,
                "tokens": n_tokens, "parallelism": f"ep{world}", "experts_per_gpu": e_local,
                "router": router,
                "max_tokens_per_expert_rank0": max(counts) if counts else 0,
                "compressed_bytes_per_gpu": store.compressed_bytes, "active_experts_rank0": active,
                "l2": f"inputs larger than L2 ({(bytes_wi + bytes_wo) / 1e6:.0f} MB of compressed experts "
                      "streamed per GPU per step)",
                "setup_s": round(setup_s, 1),
                "execution": "cuda-graph replay of the step" if gstep is not None else "eager launches",
                "eager_ms_per_step": ms_eager / args.steps,
                "pair_capacity": default_pair_capacity(t_local, world) if world > 1 else None,
                "exchange": layer.exchange if world > 1 else None,
            },
            "e2e": {"value": n_tokens * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": n_tokens * d_model * 2, "d2h_bytes_per_step": n_tokens * d_model * 2},
            "gpu_launches": int(launches),
            "roofline": {
                "kernel": "k_matmul_grouped (one launch for the work items of wi and of wo)" if fused
                          else "k_matmul_grouped (the grouped launches of wi and of wo)",
                "launches_per_step": per_step,
                "bound": "hbm", "achieved": achieved,
                "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": kernel_ms,
                "wi_ms": wi_ms.value / calls, "wo_ms": wo_ms.value / calls,
                "traffic": None if ratio is None else ratio * alg_bytes,
                "timed_in": "the eager pass before the graph capture (CUDA events around the launches on their "
                            "stream); value and e2e come from the graph replay of the same kernels",
            },
            "status": {"tile_timeouts": tile_timeouts, "exchange_overflow_tokens": overflow,
                       "peer_barrier_timeouts": peer_timeouts},
            "parity_check": parity,
            "clocks": clocks,
        }
        if kernel_times is not None:
            line["step_kernels"] = kernel_times
        if world == 1 and args.tokens_per_expert == 0 and args.experts == 0 and args.workload == "switch-c-2048":
            # the batch-1 figure: the same layer with exactly one token per expert (every one of the
            # 2048 experts active, each matrix applied to one vector), eager, event-timed launches
            lg1 = forced_logits(n_experts, n_experts).to(dev)
            h1 = synth.tokens(n_experts, d_model, SEED + 9).to(dev)
            for _ in range(2):
                full(h1, lg1)
            lib.qmoe_profile_enable(1)
            for _ in range(5):
                full(h1, lg1)
            lib.qmoe_profile_enable(0)
            _lib.check(lib.qmoe_profile_read(ctypes.byref(wi_ms), ctypes.byref(wo_ms), ctypes.byref(n_calls)))
            b1 = sum(store.matrix_bytes(m) for m in range(2 * n_experts)) / 2 + 2 * n_experts * (d_model + d_ff)
            ms1 = (wi_ms.value + wo_ms.value) / (2 * max(n_calls.value, 1))
            line["roofline_batch1"] = {
                "what": "one token per expert, all 2048 experts active: every matrix of the layer applied to one "
                        "vector in one grouped launch per linear",
                "bound": "hbm", "achieved": b1 / (ms1 * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                "frac": b1 / (ms1 * 1e-3) / 1e9 / peak, "algorithmic_bytes_per_launch": b1, "ms_per_launch": ms1}
        if world == 1:
            lg_l2 = given if given is not None else rl_chk.reshape(t_local, n_experts).float()
            ms_l2, n_l2 = l2_resident_rate(dev, d_model, d_ff, n_experts, hidden_dev, lg_l2, lib)
            gbs = (bytes_wi + bytes_wo) / (ms_l2 * 1e-3) / 1e9 if ms_l2 > 0 else None
            sm_hz = ((clocks or {}).get("sm_mhz") or 1965.0) * 1e6
            codes_step = sum(store.host_descs[2 * e].n_codes + store.host_descs[2 * e + 1].n_codes
                             for e, c in enumerate(counts) if c > 0)
            line["roofline_smem"] = {
                "bound": "smem", "achieved": achieved, "peak": gbs, "unit": "GB/s",
                "frac": achieved / gbs if gbs else None, "ms_per_step_l2_resident": ms_l2,
                "what": f"peak = this benchmark's own step (same tokens, routing and work list) on a layer whose "
                        f"{n_experts} experts alias the matrices of {n_l2} real experts, so that every code stream "
                        "stays in L2: no HBM traffic for codes, i.e. what the SMs' issue and shared-memory pipes "
                        "sustain for this decoder on this workload; achieved = the HBM-resident layer",
                "codes_per_sm_per_clock_at_peak": codes_step / (ms_l2 * 1e-3) / (148 * sm_hz) if ms_l2 > 0 else None}
        if world == 1 and not args.no_gpu_reference:
            line["gpu_reference"] = gpu_reference_leg(store, dev, d_model, d_ff, counts, hidden_dev, value)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args, d_model, d_ff, n_experts)
        print(json.dumps(line), flush=True)
    if gstep is not None:
        # NCCL keeps a communicator referenced while a CUDA graph that captured its collectives
        # exists; destroy the graph before the process group.
        torch.cuda.synchronize()
        gstep.close()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        # Teardown in a helper thread with a deadline: a run that has printed its line must not be
        # kept alive by a communicator that refuses to finalise.
        import threading
        t = threading.Thread(target=dist.destroy_process_group, daemon=True)
        t.start()
        t.join(timeout=20)
        if t.is_alive():
            sys.stderr.write(f"[bench] rank {rank}: process-group teardown did not finish; exiting\n")
            sys.stderr.flush()
            os._exit(0)


# ---------------------------------------------------------------------------------------------
# per-layer matvec latency: the reference's own benchmark (test.py:117-126,139-176)
# ---------------------------------------------------------------------------------------------
LAYER_SHAPES = [(768, 3072), (3072, 768), (1024, 4096), (4096, 1024), (2080, 6144), (6144, 2080)]


def run_layers(args):
    """One JSON line per shape.  ``--impl ours``: the new sub1matvec and the dense bf16 matvec of
    test.py:176; ``--impl reference``: the reference's own kernel built unmodified into oracle/_ref.
    Two protocols: the reference's (100 warm-up + 1000 calls, host sync after every call, wall clock)
    and back-to-back launches timed with CUDA events."""
    import torch
    from qmoe_b200 import sub1, sub1_cuda, synth
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", 0)
    ref = None
    if args.impl == "reference":
        from oracle import build_ref
        ref = build_ref.load()
        if ref is None:
            print(json.dumps({"impl": "reference", "mode": "layers",
                              "unavailable": "oracle/_ref not built (python oracle/build_ref.py)"}))
            return
    dec, trie = sub1.DEC(dev), sub1.TRIE(dev)
    iters = max(args.steps, 1) * 50

    def sync_protocol(f):
        for _ in range(100):
            f()
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            f()
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) / iters * 1e6

    def event_protocol(f):
        for _ in range(20):
            f()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            f()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e3

    for h, w in LAYER_SHAPES:
        sym = synth.ternary_cuda(h * w, SEED, synth.matrix_first_index(7 * h + w), 0.9, dev).reshape(h, w)
        codes, row_off, _, _ = sub1_cuda.sub1pack_u8(trie, sym)
        row_off = row_off[0].contiguous()
        codes = codes[: int(row_off[-1])].contiguous()
        minmax = synth.row_scales(h, SEED, 7 * h + w).to(dev)
        x = synth.tokens(1, w, SEED)[0].to(dev)
        y = torch.zeros(h, dtype=torch.bfloat16, device=dev)
        n_bytes = 2 * codes.numel() + 4 * (h + 1) + 4 * h + 2 * w + 4 * h
        line = {"mode": "layers", "impl": args.impl, "shape": [h, w], "n_codes": int(codes.numel()),
                "bits_per_weight": 16 * codes.numel() / (h * w), "algorithmic_bytes": n_bytes,
                "iters": iters, "unit": "us per call"}
        if ref is not None:
            f = lambda: ref.sub1matvec(dec, codes, row_off, minmax, x, y)  # noqa: E731
            line["sub1_sync_us"] = sync_protocol(f)
            line["sub1_events_us"] = event_protocol(f)
        else:
            f = lambda: sub1_cuda.sub1matvec(dec, codes, row_off, minmax, x, y)  # noqa: E731
            line["sub1_sync_us"] = sync_protocol(f)
            line["sub1_events_us"] = event_protocol(f)
            deq = torch.stack([torch.zeros(h, device=dev), minmax[0::2].float(), minmax[1::2].float()], 1)
            dense = torch.gather(deq, 1, sym.long()).bfloat16()
            xc, yc = x.reshape(-1, 1), torch.zeros(h, 1, dtype=torch.bfloat16, device=dev)
            g = lambda: torch.matmul(dense, xc, out=yc)  # noqa: E731
            line["dense_sync_us"] = sync_protocol(g)
            line["dense_events_us"] = event_protocol(g)
        line["sub1_gbs_events"] = n_bytes / line["sub1_events_us"] / 1e3
        print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# end-to-end greedy generation through a Switch-c-2048-shaped decoder (benchmark configuration 5)
# ---------------------------------------------------------------------------------------------
def run_generate(args):
    """15 MoE blocks of the switch-c-2048 layer with dense bf16 attention (32 heads), seeded random
    weights, batch 1: 128 prompt ids, 128 greedily generated tokens; experts sharded over the ranks
    (token stream replicated, one all-reduce per layer).  One JSON line: generated tokens/s."""
    import torch
    import torch.distributed as dist
    from qmoe_b200.decoder import SwitchDecoderLM
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    d_model, d_ff, n_experts, _ = workload_dims(args)
    layers, prompt_len, new_tokens = 15, 128, 128
    t0 = time.perf_counter()
    model = SwitchDecoderLM(d_model, d_ff, n_experts, layers, 32, 32128, prompt_len + new_tokens, dev, SEED,
                            rank, world)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t0
    prompt = torch.randint(0, 32128, (prompt_len,), generator=torch.Generator().manual_seed(SEED))
    # Teacher-forced decode input: seeded random ids, so that consecutive steps route to different
    # experts (greedy output of random weights repeats one token and would keep re-reading one expert
    # per block from L2).  --decode-input greedy feeds the argmax back instead.
    forced = None
    if args.decode_input == "forced":
        forced = torch.randint(0, 32128, (new_tokens,), generator=torch.Generator().manual_seed(SEED + 1))
    if args.decode_routing == "uniform":
        # every decode step visits a seeded random expert in every block: what a trained, balanced
        # router does to a token stream (random weights send a whole sequence to a handful of experts
        # per block, which then never leave L2)
        model.set_forced_routing(torch.randint(0, n_experts, (new_tokens, layers),
                                               generator=torch.Generator().manual_seed(SEED + 2)))
    times = []
    for it in range(max(args.steps, 1) + 1):                 # first sample is warm-up (sub1.py:382)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = model.generate(prompt, new_tokens, use_graph=not args.no_graph, forced=forced)
        torch.cuda.synchronize()
        if it > 0:
            times.append(time.perf_counter() - t0)
    secs = sum(times) / len(times)
    timing = dict(getattr(model, "last_timing", None) or {})
    # one more sample, untimed and eager, that counts which experts the decode steps visit
    model.trace_experts(True)
    model.generate(prompt, new_tokens, use_graph=False, forced=forced)
    torch.cuda.synchronize()
    trace = model.expert_trace()                               # [layers, experts]
    model.trace_experts(False)
    steps_traced = new_tokens - 1
    distinct = (trace > 0).sum(1)
    store0 = model.blocks[0]["moe"].store
    expert_bytes = sum(store0.matrix_bytes(m) for m in range(2 * store0.n_experts)) / store0.n_experts
    experts_visited = {
        "decode_steps": steps_traced, "distinct_experts_per_block_mean": float(distinct.float().mean()),
        "distinct_experts_per_block_min": int(distinct.min()), "distinct_experts_per_block_max": int(distinct.max()),
        "distinct_experts_all_blocks": int(distinct.sum()),
        "compressed_bytes_streamed_per_token": int(layers * expert_bytes),
        "note": "one expert per block and token; bytes = codes + row offsets + (min, max) of its two matrices"}
    kernel_times = None
    if args.kernel_times and world == 1:
        # five eager single-token steps under the torch profiler, after the timed samples
        from torch.profiler import ProfilerActivity, profile
        tok = out[-1:].clone()
        pos = torch.full((1,), prompt_len + new_tokens - 1, dtype=torch.int64, device=dev)
        with torch.no_grad():
            for _ in range(3):
                model.forward(tok, pos)
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(5):
                    model.forward(tok, pos)
                torch.cuda.synchronize()
        rows = [e for e in prof.key_averages() if e.device_type == torch.autograd.DeviceType.CUDA]
        total = sum(e.device_time_total for e in rows)
        kernel_times = {
            "per_step_us": round(total / 5, 1), "launches_per_step": sum(e.count for e in rows) / 5,
            "kernels": [{"name": e.key[:60], "calls_per_step": e.count / 5,
                         "avg_us": round(e.device_time_total / max(e.count, 1), 2),
                         "share": round(e.device_time_total / total, 4)}
                        for e in sorted(rows, key=lambda e: -e.device_time_total)[:12]]}
    if rank == 0:
        print(json.dumps({
            "mode": "generate", "metric": "generated_tokens_per_s", "value": new_tokens / secs, "unit": "tokens/s",
            "model": "synthetic decoder: decoder-only stand-in with the switch-c-2048 MoE blocks (scaled dot-product "
                     "attention, no relative position bias, no encoder / cross-attention); its tokens/s are not "
                     "comparable with the reference's --gentokens timing of the real encoder-decoder",
            "decode_step_kernels": kernel_times,
            "n_gpus": world, "seconds_per_sample": secs, "samples": len(times),
            "config": {"workload": args.workload + " decoder", "layers": layers, "d_model": d_model, "d_ff": d_ff,
                       "experts": n_experts, "heads": 32, "vocab": 32128, "prompt": prompt_len,
                       "generated": new_tokens, "compressed_expert_bytes_per_gpu": model.compressed_bytes,
                       "setup_s": round(setup_s, 1),
                       "execution": "eager" if args.no_graph else "cuda-graph replay of the decode step"},
            "data": "synthetic (seeded dense bf16 weights N(0,0.02), seeded ternary experts, random prompt ids)",
            "decode_input": args.decode_input, "decode_routing": args.decode_routing,
            "experts_visited": experts_visited,
            "decode_tokens_per_s": (timing["decode_steps"] / timing["decode_s"]) if timing.get("decode_s") else None,
            "timing_last_sample": timing,
            "first_tokens": out[:8].tolist()}), flush=True)
    model.close()                      # the graph holds the NCCL communicator
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def main():
    args = parse_args()
    if args.mode == "generate":
        run_generate(args)
    elif args.mode == "smem-ceiling":
        run_smem_ceiling(args)
    elif args.mode == "layers":
        run_layers(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

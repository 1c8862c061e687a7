#!/usr/bin/env python
"""Benchmark of the delta-rule hot path on B200.

Workload (per GPU): chunk_gdn2 training forward+backward at the headline shape
B=1, L=2048, Hk=12, Hv=24, K=V=128, bf16 q/k/v, fp32 gates, precision='bf16',
chunk 128, qk_l2norm, documents split at L/2, all six gradients.  Inputs are seeded
synthetic tensors with the reference benchmark's distributions.  A "step" is one
forward+backward; K steps are timed as one region between CUDA events, the region is
repeated until about half a second has been measured and the median is reported.

One JSON line is printed by rank 0:
  value        tokens/s of fwd+bwd with inputs resident in HBM, summed over all GPUs
               (every rank runs the workload on its own batch row: weak scaling); the two C-ABI calls
               of a step are captured once into a CUDA graph and replayed (`config.issue`; the
               call-by-call time is `config.call_by_call_ms_per_step`),
  e2e          the same through the public Python operator with HOST buffers (pinned H2D of
               the inputs and D2H of out + all gradients of every timed step inside the timed
               region, double-buffered); `e2e.light_inputs` is the same work with the gates
               uploaded as bf16 pre-activations (fuse_prologue), the lightest layout the operator takes,
  roofline     the slowest kernel of the step against the measured peak, plus the whole step
               against the user-visible bytes and FLOPs (`step_*` keys),
  decode       state-stream GB/s of the decode step (value heads sharded over the GPUs),
  layer_steps  the steps either side of the recurrence in a layer (conv+SiLU+split, gated RMSNorm), GB/s each,
  prefill      Gated DeltaNet packed-document forward prefill (scalar gates, B=4 L=8192, inference mode),
  sp           the long-sequence workload: KDA-style fwd+bwd on ONE packed sequence of 131072
               tokens, chunk_size 64, recompute_states, split into contiguous shards over the
               GPUs (strong scaling; the shards' affine state maps cross the ranks by one NCCL all-gather per direction),
  cpu_baseline the CPU oracle (a port of the reference's chunked path) on the host cores.

`--impl reference` times the CPU oracle on the same workload instead (the reference itself
needs an array library that is not installed on the box; the oracle restates its chunked
algorithm).  `--only chunk|decode|sp|layer` run one leg (profiling aid).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "deltanet-tpu_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

CFG = dict(B=1, L=2048, Hk=12, Hv=24, K=128, V=128, chunk=128)
DEC = dict(B=256, Hk=16, Hv=32, K=128, V=128, steps=1000)
SPCFG = dict(L=131072, H=32, K=128, V=128, chunk=64)
WORKLOAD = ("chunk_gdn2 fwd+bwd B=1 L=2048 Hk=12 Hv=24 K=V=128 chunk=128 precision=bf16 qk_l2norm, "
            "bf16 q/k/v, fp32 channel-wise gates, documents split at L/2, all six gradients")
METRIC = "chunk_gdn2 fwd+bwd tokens/s, all GPUs together (L=2048 Hk=12 Hv=24 K=V=128 bf16)"


# ------------------------------------------------------------------------------------------ peaks
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ------------------------------------------------------------------------------------------ flops and bytes
def alg_flops(c):
    """Algorithmic dense-matmul FLOPs per chunk-head of each kernel of this build.

    The terms are those of the reference kernels (prepass fwd: A and M on the lower blocks,
    the triangular inverse at C^3/3, W, U; state fwd: 3 state products + M V_new; state bwd:
    7 state products + 2 CxC products; prepass bwd) regrouped by the kernel that performs
    them here: the reverse chain keeps 3 state products + M^T dO, the chunk-parallel
    backward takes the other 4 state products + dO V_new^T and the whole prepass adjoint.
    """
    C, K, Vw = c["chunk"], c["K"], (c["Hv"] // c["Hk"]) * c["V"]
    ns = C // 32
    f = (ns + 1) / (2 * ns)
    pre_fwd = 2 * f * 2 * C * C * K + C ** 3 / 3 + 2 * C * C * K + 2 * C * C * Vw
    st_fwd = 3 * 2 * C * K * Vw + 2 * C * C * Vw
    chain_bwd = 3 * 2 * C * K * Vw + 2 * C * C * Vw
    pre_bwd_ref = 2 * 2 * C * C * K + 2 * 2 * C * C * Vw + 2 * 2 * C ** 3 + 4 * ((ns - 1) / (2 * ns)) * 2 * C * C * K
    par_bwd = 4 * 2 * C * K * Vw + 2 * C * C * Vw + pre_bwd_ref
    return dict(prepass_fwd=pre_fwd, state_fwd=st_fwd, state_bwd=chain_bwd, prepass_bwd=par_bwd)


def alg_bytes(c):
    """HBM bytes per (batch, exec head, chunk) item and kernel: every array the kernel must read or
    write, once (bf16 q/k/v/out/dO and residual tiles, fp32 gates, bf16 T / state / dV / dH images)."""
    C, K, Vw = c["chunk"], c["K"], (c["Hv"] // c["Hk"]) * c["V"]
    qk, gb, vv, ww = 2 * C * K * 2, 2 * C * K * 4, C * Vw * 2, C * Vw * 4
    tiles = 3 * C * K * 2 + C * C * 2 + C * Vw * 2              # W, qe, ke, M, U
    pre_fwd = qk + gb + vv + ww + tiles + C * C * 2 + K * 4      # + T image, Lambda_end
    st_fwd = tiles + C * Vw * 2 + K * Vw * 2                     # + out, chunk-entry state image
    chain_bwd = 3 * C * K * 2 + C * C * 2 + C * Vw * 2 + K * Vw * 2 + C * Vw * 2 + K * Vw * 2    # tiles, dO, S -> dV, dH images
    par_bwd = (C * K * 2 + C * Vw * 2 + K * Vw * 2 + C * C * 2 + C * Vw * 2 + C * Vw * 2 + K * Vw * 2
               + qk + gb + vv + ww + qk + gb + vv + ww)          # W,U,S,T,dO,dV,dH images, inputs, six gradients
    return dict(prepass_fwd=pre_fwd, state_fwd=st_fwd, state_bwd=chain_bwd, prepass_bwd=par_bwd)


def step_alg(c):
    """The whole step against what a user sees: every input read once in forward and once in backward
    in its own shape and dtype, out written, dO read, six gradients written (intermediates that go
    through HBM between the kernels are NOT counted, so they lower the fraction); dense-matmul FLOPs
    of all four kernels."""
    B, L, Hk, Hv, K, V = c["B"], c["L"], c["Hk"], c["Hv"], c["K"], c["V"]
    ins = B * L * (2 * Hk * K * 2 + Hv * V * 2 + 2 * Hk * K * 4 + Hv * V * 4)
    out = B * L * Hv * V * 2
    items = B * Hk * math.ceil(L / c["chunk"])
    return dict(bytes=3 * ins + 2 * out + 2 * B * L * 4, flops=sum(alg_flops(c).values()) * items)


def ncu_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum per kernel and step of the headline workload, taken
    from the line `traffic_bytes_per_step: kernel=bytes ...` of the kept ncu summary; {} if absent."""
    path = os.path.join(ROOT, "profiles", "chunk_step_kernels_headline.md")
    try:
        m = re.search(r"^traffic_bytes_per_step:(.*)$", open(path).read(), flags=re.M)
        return {k_: float(v_) for k_, v_ in re.findall(r"(\w+)=([0-9.eE+]+)", m.group(1))} if m else {}
    except OSError:
        return {}


# ------------------------------------------------------------------------------------------ inputs
def make_training_inputs(seed, c, device=None, pin=False, light=False):
    """light: gates as bf16 PRE-activations for fuse_prologue (sigmoid / -exp are applied in the kernels)."""
    gen = torch.Generator().manual_seed(seed)
    B, L, Hk, Hv, K, V = c["B"], c["L"], c["Hk"], c["Hv"], c["K"], c["V"]
    rn = lambda *s: torch.randn(*s, generator=gen)
    t = dict(q=rn(B, L, Hk, K).to(torch.bfloat16), k=rn(B, L, Hk, K).to(torch.bfloat16), v=rn(B, L, Hv, V).to(torch.bfloat16))
    nb, nw, ng = rn(B, L, Hk, K) * 0.39, rn(B, L, Hv, V) * 0.39, rn(B, L, Hk, K) * 0.39 - 1.0
    if light:
        t.update(b=nb.to(torch.bfloat16), w=nw.to(torch.bfloat16), g=ng.to(torch.bfloat16))
    else:
        t.update(b=torch.sigmoid(nb), w=torch.sigmoid(nw), g=-torch.exp(ng))
    t.update(do=rn(B, L, Hv, V).to(torch.bfloat16),
             seg=(torch.arange(L) >= L // 2).to(torch.int32)[None].expand(B, L).contiguous())
    if pin:
        t = {k_: v_.pin_memory() for k_, v_ in t.items()}
    if device is not None:
        t = {k_: v_.to(device) for k_, v_ in t.items()}
    return t


class DeviceJob:
    """fwd+bwd through the C ABI on pre-allocated device buffers (nothing allocated per step)."""

    def __init__(self, c, dev, seed):
        from deltanet_b200 import _lib as L
        self.L, self.lib = L, L.lib()
        self.t = make_training_inputs(seed, c, device=dev)
        t = self.t
        self.shape = L.Shape(B=c["B"], L=c["L"], Hk=c["Hk"], Hv=c["Hv"], K=c["K"], V=c["V"], chunk=c["chunk"],
                             g_heads=c["Hk"], g_cols=c["K"], b_heads=c["Hk"], b_cols=c["K"],
                             w_heads=c["Hv"], w_cols=c["V"], qkv_dtype=L.DN_BF16, gate_dtype=L.DN_F32,
                             precision=L.DN_PREC_BF16, flags=L.DN_QK_L2NORM, scale=c["K"] ** -0.5)
        self.out = torch.empty_like(t["v"])
        self.grads = {n: torch.empty_like(t[n]) for n in "qkvgbw"}
        self.res_block = torch.empty(self.lib.dn_residual_bytes(self.shape), dtype=torch.uint8, device=dev)
        self.res = L.Residuals()
        L.check(self.lib.dn_residual_carve(self.shape, self.res_block.data_ptr(), self.res), "carve")
        n = max(self.lib.dn_scratch_bytes(self.shape, 0, 0), self.lib.dn_scratch_bytes(self.shape, 1, 0))
        self.scratch = torch.empty(n, dtype=torch.uint8, device=dev)
        ex = L.Exec()
        self.lib.dn_exec_view(self.shape, ex)
        self.ex = ex
        items = c["B"] * ex.H * ex.NC
        self.dV = torch.empty(items * ex.chunk * ex.Vw, dtype=torch.float32, device=dev)
        self.dH = torch.empty(items * c["K"] * ex.Vw, dtype=torch.float32, device=dev)
        self.stream = torch.cuda.current_stream().cuda_stream
        self.bytes = sum(x.numel() * x.element_size() for x in (self.res_block, self.scratch, self.out)) + \
            sum(x.numel() * x.element_size() for x in t.values()) + \
            sum(x.numel() * x.element_size() for x in self.grads.values())

    def _p(self, n):
        return self.t[n].data_ptr()

    def fwd(self):
        L, s, sc = self.L, self.shape, self.scratch
        L.check(self.lib.dn_chunk_fwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                      self._p("w"), self._p("seg"), None, self.out.data_ptr(), None, self.res,
                                      sc.data_ptr(), sc.numel(), self.stream), "dn_chunk_fwd")

    def bwd(self):
        L, s, sc, gr = self.L, self.shape, self.scratch, self.grads
        L.check(self.lib.dn_chunk_bwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                      self._p("w"), self._p("seg"), None, self.res, self._p("do"), None,
                                      gr["q"].data_ptr(), gr["k"].data_ptr(), gr["v"].data_ptr(),
                                      gr["g"].data_ptr(), gr["b"].data_ptr(), gr["w"].data_ptr(), None,
                                      sc.data_ptr(), sc.numel(), self.stream), "dn_chunk_bwd")

    def step(self):
        self.fwd()
        self.bwd()

    # single phases, for the per-kernel timing
    def phase(self, name):
        L, s, sc = self.L, self.shape, self.scratch
        if name == "prepass_fwd":
            L.check(self.lib.dn_prepass_fwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                            self._p("w"), self._p("seg"), self.res, sc.data_ptr(), sc.numel(),
                                            self.stream), name)
        elif name == "state_fwd":
            L.check(self.lib.dn_state_fwd(s, self.res, self._p("seg"), None, self.out.data_ptr(), None, self.stream), name)
        elif name == "state_bwd":
            L.check(self.lib.dn_state_bwd(s, self.res, self._p("seg"), self._p("do"), None, self.dV.data_ptr(),
                                          self.dH.data_ptr(), None, self.stream), name)
        elif name == "prepass_bwd":
            gr = self.grads
            L.check(self.lib.dn_prepass_bwd(s, self._p("q"), self._p("k"), self._p("v"), self._p("g"), self._p("b"),
                                            self._p("w"), self._p("seg"), self.res, self._p("do"),
                                            self.dV.data_ptr(), self.dH.data_ptr(), gr["q"].data_ptr(),
                                            gr["k"].data_ptr(), gr["v"].data_ptr(), gr["g"].data_ptr(),
                                            gr["b"].data_ptr(), gr["w"].data_ptr(), sc.data_ptr(), sc.numel(),
                                            self.stream), name)


class DecodeJob:
    def __init__(self, d, dev, seed, heads=None):
        from deltanet_b200 import _lib as L
        self.L, self.lib = L, L.lib()
        Hv = heads or d["Hv"]
        Hk = max(1, Hv * d["Hk"] // d["Hv"])
        B, K, V = d["B"], d["K"], d["V"]
        gen = torch.Generator().manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=gen)
        self.q = rn(B, Hk, K).to(torch.bfloat16).to(dev)
        self.k = rn(B, Hk, K).to(torch.bfloat16).to(dev)
        self.v = rn(B, Hv, V).to(torch.bfloat16).to(dev)
        self.b = torch.sigmoid(rn(B, Hk, K) * 0.39).to(dev)
        self.w = torch.sigmoid(rn(B, Hv, V) * 0.39).to(dev)
        self.g = (-torch.exp(rn(B, Hk, K) * 0.39 - 1.0)).to(dev)
        self.state = [(torch.randn(B, Hv, K, V, device=dev) * 0.1).to(torch.bfloat16) for _ in range(2)]
        self.o = torch.empty(B, Hv, V, dtype=torch.bfloat16, device=dev)
        self.shape = L.DecodeShape(B=B, Hk=Hk, Hv=Hv, K=K, V=V, g_heads=Hk, g_cols=K, b_heads=Hk, b_cols=K,
                                   w_heads=Hv, w_cols=V, qkv_dtype=L.DN_BF16, gate_dtype=L.DN_F32,
                                   state_in_dtype=L.DN_BF16, state_out_dtype=L.DN_BF16, flags=L.DN_QK_L2NORM,
                                   scale=K ** -0.5, stability_tau=1000.0)
        self.state_bytes = 2 * B * Hv * K * V * 2
        self.vec_bytes = sum(x.numel() * x.element_size() for x in (self.q, self.k, self.v, self.b, self.w, self.g, self.o))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.i = 0

    def step(self):
        a, b_ = self.state[self.i & 1], self.state[(self.i + 1) & 1]
        self.i += 1
        self.L.check(self.lib.dn_decode_step(self.shape, self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
                                             self.g.data_ptr(), self.b.data_ptr(), self.w.data_ptr(), a.data_ptr(),
                                             None, self.o.data_ptr(), b_.data_ptr(), self.stream), "dn_decode_step")


# ------------------------------------------------------------------------------------------ helpers
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.3)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()

    def summary(self):
        sm = sorted(int(float(r[1])) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [int(float(r[2])) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for nm, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def time_steps(fn, steps, warmup, dist=None, min_seconds=0.0, max_repeats=64):
    """W warm-ups, then regions of exactly K steps between CUDA events on the current stream, repeated
    until min_seconds have been measured; returns (median region time in ms, max over ranks; repeats)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    while True:
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        more = 1.0 if (sum(times) + ms) * 1e-3 < min_seconds and len(times) + 1 < max_repeats else 0.0
        if dist is not None:
            t = torch.tensor([ms, more], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms, more = float(t[0].item()), float(t[1].item())
        times.append(ms)
        if not more:
            break
    times.sort()
    return times[len(times) // 2], len(times)


def bind_to_local_cores(local_rank, ranks_on_node):
    """Pins this process to its share of the host's cores BEFORE it allocates and first-touches its pinned
    buffers, so that they come from memory near those cores (a process setting only; no GPU or driver
    setting is involved).  Returns the number of cores now allowed."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        if ranks_on_node > 1 and len(cores) >= ranks_on_node:
            per = len(cores) // ranks_on_node
            os.sched_setaffinity(0, cores[local_rank * per:(local_rank + 1) * per])
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------ CPU oracle leg
def cpu_oracle_step(c, heads_frac=1.0, seed=11):
    """One fwd+bwd of the oracle's chunked path on the workload (or a head-subset of it); returns seconds."""
    from oracle import delta_oracle as O
    Hk = max(1, int(round(c["Hk"] * heads_frac)))
    Hv = Hk * (c["Hv"] // c["Hk"])
    cc = dict(c, Hk=Hk, Hv=Hv)
    t = make_training_inputs(seed, cc)
    ins = [t[n].clone().requires_grad_() for n in "qkvgbw"]
    t0 = time.perf_counter()
    o = O.chunk_gdn2(*ins, segment_ids=t["seg"], chunk_size=c["chunk"], precision="bf16", qk_l2norm=True)
    torch.autograd.grad((o.float() * t["do"].float()).sum(), ins)
    return time.perf_counter() - t0, Hv / c["Hv"]


def run_reference(args):
    """The CPU arm: the oracle port of the reference's chunked forward + backward on the SAME workload,
    all 24 value heads per step, on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    times, budget, t_start = [], 240.0, time.perf_counter()
    cpu_oracle_step(CFG, 1.0 / 12.0)                           # first-call overheads
    cpu_oracle_step(CFG)                                       # one full-size warm-up step is enough on a CPU
    while len(times) < args.steps:
        if times and time.perf_counter() - t_start > budget:
            break
        times.append(cpu_oracle_step(CFG)[0])
    sec = sorted(times)[len(times) // 2]
    tok = CFG["B"] * CFG["L"] / sec
    sample = (f"oracle port of the reference's chunked path (gdn2.py:772-1173), torch CPU, {cores} threads; each step = "
              f"fwd+bwd on the whole workload (24 of 24 value heads, L=2048); median of {len(times)} timed steps")
    line = dict(metric=METRIC, value=tok, unit="tokens/s",
                impl="reference", n_gpus=args.gpus, steps=len(times), warmup=args.warmup, ms_per_step=sec * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                config=dict(workload=WORKLOAD),
                cpu_baseline=dict(value=tok, unit="tokens/s", cores=cores, kind="port", sample=sample),
                e2e=dict(value=tok, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ long sequence
def sp_leg(dn, dist, world, rank, dev, steps=3):
    """KDA-style fwd+bwd on ONE packed sequence of 131072 tokens (channel-wise decay, per-head beta,
    documents of 2048..32768 tokens, chunk_size 64, recompute_states), split into equal contiguous
    shards over the ranks: the shards' affine state maps cross the ranks in one NCCL all-gather per direction, everything else is
    local.  Total work is fixed, so this is strong scaling.  Returns the `sp` object (rank 0) or None."""
    from deltanet_b200 import sp
    c = SPCFG
    L, H, K, V = c["L"], c["H"], c["K"], c["V"]
    gen = torch.Generator().manual_seed(4000)
    lens, tot = [], 0
    while tot < L:
        n = int(torch.randint(2048, 32769, (1,), generator=gen))
        lens.append(min(n, L - tot))
        tot += lens[-1]
    seg = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int32), torch.tensor(lens))[None]

    def make(lo, hi, seed):
        g2 = torch.Generator(device=dev).manual_seed(seed)
        rn = lambda *sh: torch.randn(*sh, generator=g2, device=dev)
        n = hi - lo
        return dict(q=rn(1, n, H, K).bfloat16().requires_grad_(), k=rn(1, n, H, K).bfloat16().requires_grad_(),
                    v=rn(1, n, H, V).bfloat16().requires_grad_(), g=(-torch.exp(rn(1, n, H, K) * 0.39 - 1.0)).requires_grad_(),
                    beta=torch.sigmoid(rn(1, n, H)).requires_grad_(), do=rn(1, n, H, V).bfloat16(),
                    seg=seg[:, lo:hi].contiguous().to(dev))

    def run(t, sharded):
        if sharded:
            o, _ = sp.chunk_gdn2_sp(t["q"], t["k"], t["v"], t["g"], t["beta"], t["beta"], segment_ids=t["seg"],
                                    chunk_size=c["chunk"], precision="bf16", qk_l2norm=True, recompute_states=True)
        else:
            o = dn.chunk_kda(t["q"], t["k"], t["v"], t["g"], t["beta"], segment_ids=t["seg"], chunk_size=c["chunk"],
                             qk_l2norm=True, recompute_states=True)
        torch.autograd.grad(o, [t["q"], t["k"], t["v"], t["g"], t["beta"]], grad_outputs=t["do"])

    lib = dn._lib.lib()
    mine = make(rank * L // world, (rank + 1) * L // world, 4100 + rank)
    n0 = lib.dn_launches_total()
    ms, reps = time_steps(lambda: run(mine, world > 1), steps, 3, dist)
    launches = (lib.dn_launches_total() - n0) // (reps * steps + 3)
    ms /= steps
    del mine
    single_ms = None
    if world > 1:                                               # the same sequence on ONE GPU of this box, for the ratio
        if rank == 0:
            torch.cuda.empty_cache()
            whole = make(0, L, 4100)
            single_ms = time_steps(lambda: run(whole, False), steps, 2)[0] / steps
            del whole
            torch.cuda.empty_cache()
        dist.barrier()
    if rank != 0:
        return None
    out = dict(workload="chunk_kda fwd+bwd B=1 L=131072 H=32 K=V=128 chunk_size=64 bf16 qk_l2norm recompute_states, "
                        "documents of 2048..32768 tokens (seeded), one sequence",
               parallelism=(f"sequence-sharded x{world}: per-shard affine summary, ONE NCCL all-gather of the shards' "
                            "affine maps per direction (each rank composes its predecessors' maps), partial correction pass")
               if world > 1 else "one GPU",
               scaling="strong", ms_per_step=ms, tokens_per_s=L / (ms * 1e-3), steps=steps, warmup=3,
               kernels_per_step_per_rank=int(launches))
    if single_ms is not None:
        out.update(single_gpu_ms_per_step=single_ms, speedup_vs_single_gpu=single_ms / ms,
                   efficiency_vs_single_gpu=single_ms / ms / world)
    return out


# ------------------------------------------------------------------------------------------ packed prefill
def prefill_leg(dn, dev):
    """Gated DeltaNet packed-document forward prefill through the public operator (`chunk_gdn`, is_inference,
    final state returned): B=4, L=8192, Hk=16, Hv=32, K=V=128, bf16 q/k/v, one fp32 decay and beta per (token,
    value head), document lengths geometric with mean 1024 clipped to >= 32 (seeded).  Device-resident inputs."""
    B, L, Hk, Hv, K, V = 4, 8192, 16, 32, 128, 128
    gen = torch.Generator().manual_seed(6000)
    seg = torch.empty(B, L, dtype=torch.int32)
    for b in range(B):
        t, d = 0, 0
        while t < L:
            n = max(32, int(torch.empty(1).geometric_(1.0 / 1024.0, generator=gen)))
            seg[b, t:t + n] = d
            t, d = t + n, d + 1
    g2 = torch.Generator(device=dev).manual_seed(6001)
    rn = lambda *sh: torch.randn(*sh, generator=g2, device=dev)
    q, k, v = rn(B, L, Hk, K).bfloat16(), rn(B, L, Hk, K).bfloat16(), rn(B, L, Hv, V).bfloat16()
    A = 1 + 15 * torch.rand(Hv, generator=g2, device=dev)
    g = -A * torch.nn.functional.softplus(rn(B, L, Hv) + 0.5 * rn(Hv))
    beta = torch.sigmoid(rn(B, L, Hv))
    seg = seg.to(dev)
    lib = dn._lib.lib()
    fn = lambda: dn.chunk_gdn(q, k, v, g, beta, segment_ids=seg, is_inference=True, output_final_state=True, qk_l2norm=True)
    n0 = lib.dn_launches_total()
    ms, reps = time_steps(fn, 5, 3, min_seconds=0.1)
    launches = (lib.dn_launches_total() - n0) // (reps * 5 + 3)
    ms /= 5
    in_bytes = (q.numel() + k.numel() + v.numel()) * 2 + (g.numel() + beta.numel()) * 4 + seg.numel() * 4
    out_bytes = v.numel() * 2 + B * Hv * K * V * 4
    return dict(workload="chunk_gdn forward prefill, is_inference, B=4 L=8192 Hk=16 Hv=32 K=V=128 bf16 qk_l2norm, scalar gates per "
                         "(token, value head), documents geometric(mean 1024) >= 32 tokens, final state returned",
                ms_per_step=ms, tokens_per_s=B * L / (ms * 1e-3), user_mbytes=round((in_bytes + out_bytes) / 1e6, 1),
                user_gbs=(in_bytes + out_bytes) / (ms * 1e-3) / 1e9, kernels_per_step=int(launches))


# ------------------------------------------------------------------------------------------ layer steps
def layer_steps_leg(dn, dev, peaks):
    """The steps either side of the recurrence at the packed-prefill layer shape (B=4, L=8192, Hk=16, Hv=32,
    K=V=128, bf16, conv width 4): each kernel alone, achieved HBM GB/s on the bytes it must move (inputs read
    once, outputs written once) against the measured copy bandwidth.  Device-resident buffers, C ABI."""
    from deltanet_b200 import _lib as L
    lib = L.lib()
    B, Lq, Hk, Hv, K, V, W = 4, 8192, 16, 32, 128, 128, 4
    D = 2 * Hk * K + Hv * V
    rows = B * Lq * Hv
    gen = torch.Generator(device=dev).manual_seed(5000)
    rn = lambda *sh: torch.randn(*sh, generator=gen, device=dev)
    mixed, d_mixed = rn(B, Lq, D).bfloat16(), torch.empty(B, Lq, D, dtype=torch.bfloat16, device=dev)
    w, dw, db = rn(D, W) * 0.5, torch.empty(D, W, device=dev), torch.empty(D, device=dev)
    q, k = (torch.empty(B, Lq, Hk, K, dtype=torch.bfloat16, device=dev) for _ in range(2))
    v = torch.empty(B, Lq, Hv, V, dtype=torch.bfloat16, device=dev)
    z, y = rn(B, Lq, Hv, V).bfloat16(), torch.empty(B, Lq, Hv, V, dtype=torch.bfloat16, device=dev)
    d_o, d_z = torch.empty_like(y), torch.empty_like(y)
    nw, dnw = 1 + 0.2 * rn(V), torch.empty(V, device=dev)
    seg = (torch.arange(Lq, device=dev) // 1024).to(torch.int32)[None].expand(B, Lq).contiguous()
    sc1 = torch.empty(lib.dn_gdn_producer_scratch_bytes(B, Lq, D, W), dtype=torch.uint8, device=dev)
    sc2 = torch.empty(lib.dn_gated_rmsnorm_scratch_bytes(rows, V), dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    P = lambda t: t.data_ptr()
    calls = dict(
        producer_fwd=(lambda: L.check(lib.dn_gdn_producer_fwd(P(mixed), P(w), None, P(seg), B, Lq, Hk, Hv, K, V, W, L.DN_BF16,
                                                            P(q), P(k), P(v), st), "producer_fwd"), 2 * mixed.numel() * 2),
        producer_bwd=(lambda: L.check(lib.dn_gdn_producer_bwd(P(mixed), P(w), None, P(seg), B, Lq, Hk, Hv, K, V, W, L.DN_BF16,
                                                            P(q), P(k), P(v), P(d_mixed), P(dw), None, P(sc1), sc1.numel(), st),
                                      "producer_bwd"), 3 * mixed.numel() * 2),
        gated_rmsnorm_fwd=(lambda: L.check(lib.dn_gated_rmsnorm_fwd(P(v), P(z), P(nw), rows, V, L.DN_BF16, 1e-6, P(y), st),
                                           "norm_fwd"), 3 * y.numel() * 2),
        gated_rmsnorm_bwd=(lambda: L.check(lib.dn_gated_rmsnorm_bwd(P(v), P(z), P(nw), rows, V, L.DN_BF16, 1e-6, P(y), P(d_o),
                                                                  P(d_z), P(dnw), P(sc2), sc2.numel(), st), "norm_bwd"),
                           5 * y.numel() * 2),
    )
    out = dict(workload="GDN layer steps at B=4 L=8192 Hk=16 Hv=32 K=V=128 bf16, conv width 4, documents of 1024 tokens", kernels={})
    for name, (fn, nbytes) in calls.items():
        ms = time_steps(fn, 10, 3, min_seconds=0.05)[0] / 10
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["kernels"][name] = dict(ms=round(ms, 4), alg_mbytes=round(nbytes / 1e6, 1), gbs=round(gbs, 1),
                                    frac=round(gbs / peaks["hbm_gbs"], 3))
    return out


# ------------------------------------------------------------------------------------------ end to end
def e2e_leg(dn, dev, dist, world, rank, steps, light):
    """fwd+bwd through the public operator from pinned HOST buffers, every step's uploads and read-backs
    inside the timed region: serial, and double-buffered over a copy-in stream, the compute stream and a
    copy-out stream as a training loop prefetches."""
    tokens = CFG["B"] * CFG["L"]
    host = make_training_inputs(2000 + rank, CFG, pin=True, light=light)
    names = "qkvgbw"
    in_names = list(names) + ["do", "seg"]
    h2d = sum(host[n].numel() * host[n].element_size() for n in in_names)
    out_host = {n: torch.empty_like(host[n]).pin_memory() for n in names}
    o_host = torch.empty_like(host["v"]).pin_memory()
    for t in list(out_host.values()) + [o_host]:
        t.zero_()                                              # first touch from this process's cores
    d2h = sum(host[n].numel() * host[n].element_size() for n in names) + o_host.numel() * o_host.element_size()
    kw = dict(chunk_size=CFG["chunk"], precision="bf16", qk_l2norm=True, fuse_prologue=light)

    def serial_step():
        d = {n: host[n].to(dev, non_blocking=True) for n in in_names}
        ins = [d[n].requires_grad_() for n in names]
        o = dn.chunk_gdn2(*ins, segment_ids=d["seg"], **kw)
        grads = torch.autograd.grad(o, ins, grad_outputs=d["do"])
        o_host.copy_(o.detach(), non_blocking=True)
        for n, gr in zip(names, grads):
            out_host[n].copy_(gr, non_blocking=True)

    ms_serial = time_steps(serial_step, steps, 3, dist)[0] / steps

    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    slots = [{n: torch.empty_like(host[n], device=dev) for n in in_names} for _ in range(2)]
    loaded = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(freed[i % 2])
            for n in in_names:
                slots[i % 2][n].copy_(host[n], non_blocking=True)
            loaded[i % 2].record(s_in)

    def run_pipeline(k):
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        upload(0)
        for i in range(k):
            if i + 1 < k:
                upload(i + 1)
            d = slots[i % 2]
            main.wait_event(loaded[i % 2])
            ins = [d[n].detach().requires_grad_() for n in names]
            o = dn.chunk_gdn2(*ins, segment_ids=d["seg"], **kw)
            grads = torch.autograd.grad(o, ins, grad_outputs=d["do"])
            freed[i % 2].record(main)
            s_out.wait_stream(main)
            with torch.cuda.stream(s_out):
                o_host.copy_(o.detach(), non_blocking=True)
                o.record_stream(s_out)
                for n, gr in zip(names, grads):
                    out_host[n].copy_(gr, non_blocking=True)
                    gr.record_stream(s_out)
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    ms = time_steps(lambda: run_pipeline(steps), 1, 1, dist, min_seconds=0.3, max_repeats=8)[0] / steps
    return dict(value=world * tokens / (ms * 1e-3), unit="tokens/s", ms_per_step=ms, h2d_bytes_per_step=h2d,
                d2h_bytes_per_step=d2h, unpipelined_ms_per_step=ms_serial,
                host_gbs_per_rank=(h2d + d2h) / (ms * 1e-3) / 1e9)


# ------------------------------------------------------------------------------------------ main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="repeat the timed region of K steps until this much time has been measured (0: one region)")
    ap.add_argument("--only", default="all", choices=["all", "chunk", "decode", "sp", "layer"],
                    help="profiling aid: run only the chunked fwd+bwd device loop, only the decode loop, only the long-sequence leg, or only the layer steps")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    host_cores = bind_to_local_cores(local, int(os.environ.get("LOCAL_WORLD_SIZE", str(world))))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod
    import deltanet_b200 as dn
    lib = dn._lib.lib()
    peaks = measured_peaks()
    tokens = CFG["B"] * CFG["L"]

    if args.only == "sp":
        r = sp_leg(dn, dist, world, rank, dev, steps=max(2, min(args.steps, 5)))
        if rank == 0:
            print(json.dumps(dict(only="sp", n_gpus=world, **r)), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return
    if args.only == "layer":
        if rank == 0:
            print(json.dumps(dict(only="layer", **layer_steps_leg(dn, dev, peaks))), flush=True)
        return
    if args.only == "decode":
        dj = DecodeJob(DEC, dev, seed=3000 + rank, heads=DEC["Hv"] // world)
        ms_dec = time_steps(dj.step, args.steps, args.warmup, dist)[0] / args.steps
        if rank == 0:
            print(json.dumps(dict(only="decode", us_per_step=ms_dec * 1e3,
                                  state_gbs=world * dj.state_bytes / (ms_dec * 1e-3) / 1e9)), flush=True)
        return
    # ---- device-resident throughput through the C ABI
    job = DeviceJob(CFG, dev, seed=1000 + rank)
    n0 = lib.dn_launches_total()
    with ClockSampler(local) as clk:
        ms, repeats = time_steps(job.step, args.steps, args.warmup, dist, min_seconds=args.min_seconds)
    launches_per_region = (lib.dn_launches_total() - n0) * args.steps // (args.warmup + repeats * args.steps)
    clocks = clk.summary()
    ms_step = ms / args.steps
    value = world * tokens / (ms_step * 1e-3)

    if args.only == "chunk":
        if rank == 0:
            print(json.dumps(dict(only="chunk", ms_per_step=ms_step, tokens_per_s=value, repeats=repeats)), flush=True)
        return
    # ---- the same two C-ABI calls captured ONCE into a CUDA graph and replayed: the eight launches and the
    #      fork / join of the library's side stream become graph nodes, which takes the launch gaps between
    #      dependent kernels out of a 0.36 ms step.  This is what `value` reports; the call-by-call time stays
    #      in `config`.
    call_by_call_ms = ms_step
    issue = "dn_chunk_fwd + dn_chunk_bwd captured once into a CUDA graph, replayed per step"
    main_stream_handle = job.stream
    try:
        cap_stream = torch.cuda.Stream(device=dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap_stream):
            job.stream = cap_stream.cuda_stream
            job.step()
            torch.cuda.synchronize()
            n_cap = lib.dn_launches_total()
            with torch.cuda.graph(graph, stream=cap_stream):
                job.step()
            launches_per_step = lib.dn_launches_total() - n_cap
        job.stream = main_stream_handle
        torch.cuda.synchronize()
        with ClockSampler(local) as clk:
            ms, repeats = time_steps(graph.replay, args.steps, args.warmup, dist, min_seconds=args.min_seconds)
        clocks = clk.summary()
        ms_step = ms / args.steps
        value = world * tokens / (ms_step * 1e-3)
        launches_per_region = launches_per_step * args.steps
    except RuntimeError as e:                                  # capture refused on this box: the call-by-call numbers stand
        job.stream = main_stream_handle
        torch.cuda.synchronize()
        issue = f"call by call (stream capture failed: {str(e).splitlines()[0][:120]})"
    # ---- per-kernel timing (each kernel alone, CUDA events on its stream) and the roofline of the slowest
    fl = alg_flops(CFG)
    items = CFG["B"] * job.ex.H * job.ex.NC
    job.step()
    per = {}
    for name in ("prepass_fwd", "state_fwd", "state_bwd", "prepass_bwd"):
        per[name] = time_steps(lambda: job.phase(name), 20, 3, min_seconds=0.05)[0] / 20
    dom = max(per, key=per.get)
    by = alg_bytes(CFG)
    t_hbm = by[dom] * items / (peaks["hbm_gbs"] * 1e9)          # seconds at the measured copy bandwidth
    t_tc = fl[dom] * items / (peaks["bf16_tflops"] * 1e12)      # seconds at the measured dense bf16 rate
    sec = per[dom] * 1e-3
    if t_hbm >= t_tc:
        ach = by[dom] * items / sec / 1e9
        roofline = dict(kernel=dom, bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"])
    else:
        ach = fl[dom] * items / sec / 1e12
        roofline = dict(kernel=dom, bound="tensor", achieved=ach, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                        frac=ach / peaks["bf16_tflops"])
    st = step_alg(CFG)
    st_hbm, st_tc = st["bytes"] / (peaks["hbm_gbs"] * 1e9), st["flops"] / (peaks["bf16_tflops"] * 1e12)
    traffic = ncu_traffic()
    roofline.update(traffic=traffic.get(dom), peak_source=peaks["source"],
                    tensor_frac=fl[dom] * items / sec / 1e12 / peaks["bf16_tflops"],
                    hbm_frac=by[dom] * items / sec / 1e9 / peaks["hbm_gbs"],
                    kernel_ms={k_: round(v_, 4) for k_, v_ in per.items()},
                    alg_gflop={k_: round(v_ * items / 1e9, 3) for k_, v_ in fl.items()},
                    alg_mbytes={k_: round(v_ * items / 1e6, 1) for k_, v_ in by.items()},
                    step_alg_mbytes=round(st["bytes"] / 1e6, 1), step_alg_gflop=round(st["flops"] / 1e9, 2),
                    step_bound="hbm" if st_hbm >= st_tc else "tensor",
                    step_frac=max(st_hbm, st_tc) / (ms_step * 1e-3),
                    step_traffic=sum(traffic.values()) or None)

    # ---- end to end through the public operator with host buffers
    e2e_steps = max(3, min(args.steps, 40))
    e2e = e2e_leg(dn, dev, dist, world, rank, e2e_steps, light=False)
    e2e.update(schedule="double-buffered: upload of batch i+1 and read-back of batch i-1 overlap batch i",
               host_cores_per_rank=host_cores,
               light_inputs=dict(layout="gates as bf16 pre-activations, fuse_prologue=True (sigmoid / -exp in the kernels)",
                                 **e2e_leg(dn, dev, dist, world, rank, e2e_steps, light=True)))

    # ---- decode: value heads sharded over the ranks, no collective
    dj = DecodeJob(DEC, dev, seed=3000 + rank, heads=DEC["Hv"] // world)
    dsteps = DEC["steps"]
    # a serving loop replays its decode steps from a CUDA graph: 50 consecutive calls of dn_decode_step (state
    # ping-pong between two buffers) are captured once and replayed dsteps / 50 times
    per_graph = 50
    dec_issue = f"{per_graph} consecutive dn_decode_step calls captured into a CUDA graph, replayed {dsteps // per_graph} times"
    dec_stream_handle = dj.stream
    try:
        dstream, dgraph = torch.cuda.Stream(device=dev), torch.cuda.CUDAGraph()
        with torch.cuda.stream(dstream):
            dj.stream = dstream.cuda_stream
            dj.step()
            dj.step()
            torch.cuda.synchronize()
            with torch.cuda.graph(dgraph, stream=dstream):
                for _ in range(per_graph):
                    dj.step()
        torch.cuda.synchronize()
        ms_dec = time_steps(dgraph.replay, dsteps // per_graph, 2, dist)[0] / dsteps
    except RuntimeError as e:
        dj.stream = dec_stream_handle
        torch.cuda.synchronize()
        dec_issue = f"call by call (stream capture failed: {str(e).splitlines()[0][:120]})"
        ms_dec = time_steps(dj.step, dsteps, 20, dist)[0] / dsteps
    st_gbs = world * dj.state_bytes / (ms_dec * 1e-3) / 1e9
    decode = dict(workload=f"gdn2 decode step, 256 sequences, Hk=16 Hv=32 K=V=128, bf16 state, {DEC['Hv'] // world} value heads per GPU",
                  us_per_step=ms_dec * 1e3, state_gbs=st_gbs,
                  total_gbs=world * (dj.state_bytes + dj.vec_bytes) / (ms_dec * 1e-3) / 1e9, steps=dsteps,
                  issue=dec_issue,
                  roofline=dict(bound="hbm", achieved=st_gbs / world, peak=peaks["hbm_gbs"], unit="GB/s",
                                frac=st_gbs / world / peaks["hbm_gbs"], traffic=None, peak_source=peaks["source"]))
    touched_mb = job.bytes / 1e6
    del dj, job
    torch.cuda.empty_cache()

    # ---- the layer steps either side of the path (one GPU's worth; rank 0 reports)
    layer = layer_steps_leg(dn, dev, peaks) if rank == 0 else None
    torch.cuda.empty_cache()
    prefill = prefill_leg(dn, dev) if rank == 0 else None
    torch.cuda.empty_cache()

    # ---- the long-sequence workload, sharded over the ranks
    spr = sp_leg(dn, dist, world, rank, dev)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        cpu_oracle_step(CFG, 1.0 / 12.0)                       # warm-up on a small slice
        sec, _ = cpu_oracle_step(CFG)
        cpu = dict(value=tokens / sec, unit="tokens/s", cores=cores, kind="port",
                   sample=f"CPU oracle (port of the reference's chunked fwd+bwd, gdn2.py:772-1173), one step on the whole "
                          f"workload (24 of 24 value heads, L=2048), {sec:.1f} s")
    line = dict(
        metric=METRIC, value=value, unit="tokens/s",
        n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload=WORKLOAD, global_batch=world, parallelism=f"batch-sharded x{world}, no collective",
                    timing=f"median of {repeats} regions of {args.steps} steps",
                    issue=issue,
                    call_by_call_ms_per_step=call_by_call_ms,
                    l2=f"no flush: the step touches {touched_mb:.0f} MB (inputs, residuals, scratch, grads) > 126 MB L2"),
        roofline=roofline, e2e=e2e, decode=decode, sp=spr, prefill=prefill, layer_steps=layer, cpu_baseline=cpu,
        gpu_launches=int(launches_per_region), clocks=clocks)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

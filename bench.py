#!/usr/bin/env python
"""Benchmark of the chunked gated delta rule on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload train|fwd]

One "step" is one forward + backward pass of chunk_gated_delta_rule over one synthetic batch of the
headline shape (B=4, T=4096, H=HV=16, K=V=128, bf16 q/k/v, fp32 g/beta, fp32 initial state): forward
call + ``o.backward(do)``, the reference's own definition (benchmarks/ops/run.py:246-255).  With
N > 1 (launched by torch.distributed.run) every rank processes its own batch of that shape
(heads/batch shard with no communication: weak scaling) and the value is the sum over ranks divided
by the slowest rank's time.  Prints ONE JSON line.

``--impl reference`` times the CPU restatement of the reference's naive recurrence (oracle/) on a
bounded sample of the same workload on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, 'flash-linear-attention_b200')
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

METRIC = 'tokens/s chunk_gated_delta_rule fwd+bwd (B4 T4096 H16 D128 bf16); % tensor peak'
B, T, H, HV, K, V, BT = 4, 4096, 16, 16, 128, 128, 64

# algorithmic FLOPs per (token, value head), dense-tile counting, no recomputation
STAGE_FLOPS = {
    'intra_fwd': 2 * BT * (2 * K + V),
    'scan_fwd': 4 * K * V,
    'out_fwd': 2 * K * V + 2 * BT * (K + V),
    'dv_local': 2 * BT * (K + V),
    'scan_bwd': 6 * K * V,
    'bwd_dqk': 4 * K * V + 2 * BT * (V + 2 * K),                       # dP, do h^T, v dh^T, dP k, dP^T q
    'bwd_wy': 2 * K * V + 2 * BT * (5 * K + 2 * V + 2 * BT),           # dv2 h^T + WY backward
}


def stage_bytes(R, C, NS):
    """Algorithmic HBM bytes of every kernel of one fwd+bwd step: each operand read once, each result written
    once (R token rows, C chunks, NS sequences; bf16 tiles, fp32 gates / row vectors / dk partials)."""
    qk, wv = R * H * K * 2, R * HV * V * 2           # q or k ; v, u, v_new, do, dv2, o, dv
    w = R * HV * K * 2
    a_ = R * HV * BT * 2
    snap = C * HV * K * V * 2                         # h or dh snapshots
    st32 = NS * HV * K * V * 4                        # h0, ht, dht, dh0
    gam, vec = C * HV * BT * 4, R * HV * 4
    dkp = R * H * K * 2                               # chunk-local part of dk, bf16, passed through the dk buffer
    return {
        'intra_fwd': qk + wv + 2 * vec + a_ + w + wv + gam,
        'scan_fwd': w + qk + wv + gam + st32 + snap + wv + st32,
        'out_fwd': 2 * qk + wv + snap + gam + wv,
        'dv_local': 2 * qk + wv + gam + wv,
        'scan_bwd': 2 * qk + w + 2 * wv + gam + st32 + wv + snap + st32,
        'bwd_dqk': 2 * qk + 2 * wv + 2 * snap + gam + qk + dkp + vec,
        'bwd_wy': qk + 2 * wv + a_ + snap + gam + 2 * vec + dkp + qk + wv + 2 * vec,
    }


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the headline workload, from one ncu
# capture of this script on a B200 (summary kept under profiles/); a kernel missing here was not captured.
NCU_TRAFFIC_BYTES = {
    'intra_fwd': 256.8e6, 'scan_fwd': 364.1e6, 'out_fwd': 388.7e6, 'dv_local': 244.2e6,
    'scan_bwd': 507.2e6, 'bwd_dqk': 654.0e6, 'bwd_wy': 553.0e6,
}

F_FWD = sum(STAGE_FLOPS[s] for s in ('intra_fwd', 'scan_fwd', 'out_fwd'))
F_BWD = sum(STAGE_FLOPS[s] for s in ('dv_local', 'scan_bwd', 'bwd_dqk', 'bwd_wy'))
assert F_FWD == 180224 and F_BWD == 409600


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16=p['bf16_tflops'], bf16_sustained=p.get('bf16_tflops_sustained', p['bf16_tflops']),
                    hbm=p['hbm_gbs'], source='measured')
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source='fallback')


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
         'clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits', '-lms', '100', '-i', str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['nvidia-smi unavailable'])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(',')]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), f[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['no samples'])
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        return dict(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


def make_batch(seed, device=None, pin=False):
    """Synthetic inputs with the distributions of the headline configuration (seeded, generated on the host):
    q, k ~ N(0,1) L2-normalised over K; v, do ~ N(0,1); g = logsigmoid(N(0,1)); beta = sigmoid(N(0,1));
    initial state ~ N(0, 0.1^2) fp32 (benchmarks/ops/registry.py:323-335 of the reference)."""
    gen = torch.Generator().manual_seed(seed)
    nrm = torch.nn.functional.normalize
    out = {
        'q': nrm(torch.randn(B, T, H, K, generator=gen), p=2, dim=-1).to(torch.bfloat16),
        'k': nrm(torch.randn(B, T, H, K, generator=gen), p=2, dim=-1).to(torch.bfloat16),
        'v': torch.randn(B, T, HV, V, generator=gen).to(torch.bfloat16),
        'g': torch.nn.functional.logsigmoid(torch.randn(B, T, HV, generator=gen)),
        'beta': torch.sigmoid(torch.randn(B, T, HV, generator=gen)),
        'h0': torch.randn(B, HV, K, V, generator=gen) * 0.1,
        'do': torch.randn(B, T, HV, V, generator=gen).to(torch.bfloat16),
    }
    if pin:
        out = {n: x.pin_memory() for n, x in out.items()}
    if device is not None:
        out = {n: x.to(device) for n, x in out.items()}
    return out


def step_device(batch, op):
    leaves = [batch[n].detach().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
    o, _ = op(*leaves, initial_state=batch['h0'], output_final_state=True)
    o.backward(batch['do'])
    return o, leaves


def time_stages(batch, steps):
    """Average device time of every kernel of one fwd+bwd step, CUDA events on the launching stream."""
    from b200gdn import _lib
    from b200gdn.chunk import new_chunk_args
    from b200gdn.index import tables_for
    dev = batch['q'].device
    tables = tables_for(B, T, None, None, dev)
    n_chunks, n_seq = tables[2]
    rows = B * T
    bf = dict(dtype=torch.bfloat16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    buf = dict(o=torch.empty(rows, HV, V, **bf), ht=torch.empty(n_seq, HV, K, V, **f32), gamma=torch.empty(n_chunks, HV, 64, **f32),
               A=torch.empty(rows, HV, 64, **bf), w=torch.empty(rows, HV, K, **bf), u=torch.empty(rows, HV, V, **bf),
               h=torch.empty(n_chunks, HV, K, V, **bf), v_new=torch.empty(rows, HV, V, **bf),
               dq=torch.empty(rows, H, K, **bf), dk=torch.empty(rows, H, K, **bf), dv=torch.empty(rows, HV, V, **bf),
               dg=torch.empty(rows, HV, **f32), dbeta=torch.empty(rows, HV, **f32), dh0=torch.empty(n_seq, HV, K, V, **f32),
               dh=torch.empty(n_chunks, HV, K, V, **bf), dv2=torch.empty(rows, HV, V, **bf),
               dG=torch.empty(rows, HV, **f32))
    a = new_chunk_args(batch['q'], batch['k'], batch['v'], K ** -0.5, tables)
    a.g, a.beta, a.h0 = batch['g'].data_ptr(), batch['beta'].data_ptr(), batch['h0'].data_ptr()
    a.d_o = batch['do'].data_ptr()
    for n, x in buf.items():
        setattr(a, n, x.data_ptr())
    stream = torch.cuda.current_stream(dev)
    plan = [('intra_fwd', 'b200gdn_chunk_fwd', _lib.FWD_INTRA), ('scan_fwd', 'b200gdn_chunk_fwd', _lib.FWD_SCAN),
            ('out_fwd', 'b200gdn_chunk_fwd', _lib.FWD_OUT), ('dv_local', 'b200gdn_chunk_bwd', _lib.BWD_DVLOCAL),
            ('scan_bwd', 'b200gdn_chunk_bwd', _lib.BWD_SCAN), ('bwd_dqk', 'b200gdn_chunk_bwd', _lib.BWD_DQKWG),
            ('bwd_wy', 'b200gdn_chunk_bwd', _lib.BWD_WY)]
    total = {n: 0.0 for n, _, _ in plan}
    for it in range(steps + 1):
        evs = []
        for name, fn, mask in plan:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.stage_mask = mask
            e0.record(stream)
            _lib.call(fn, a, stream.cuda_stream)
            e1.record(stream)
            evs.append((name, e0, e1))
        torch.cuda.synchronize(dev)
        if it == 0:
            continue  # warm-up
        for name, e0, e1 in evs:
            total[name] += e0.elapsed_time(e1)
    return {n: t / steps for n, t in total.items()}


def cpu_baseline(seconds_budget=20.0, threads=None):
    """The oracle's naive recurrence, forward + backward by autograd, on a bounded slice of the headline
    workload (same K, V, distributions; fewer tokens and heads), on the host cores."""
    from oracle.gdn_oracle import make_inputs, naive_recurrent
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    Bs, Ts, Hs = 1, 1024, 4
    d = make_inputs(Bs, Ts, Hs, Hs, K, V, seed=0)

    def one():
        leaves = [d[n].clone().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
        o, ht = naive_recurrent(*leaves, scale=K ** -0.5, initial_state=d['h0'], output_final_state=True)
        (o * d['do']).sum().backward()
    t0 = time.perf_counter()
    one()
    first = time.perf_counter() - t0
    reps = max(1, min(8, int(seconds_budget / max(first, 1e-3)) - 1))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one()
        times.append(time.perf_counter() - t0)
    t = statistics.median(times) if times else first
    # tokens/s of the full 16-head workload = token-heads per second / 16
    value = (Bs * Ts * Hs / HV) / t
    sample = (f'naive recurrence fwd+bwd (autograd), B={Bs} T={Ts} H=HV={Hs} K=V={K} fp32, median of {max(reps, 1)} runs of '
              f'{t:.2f} s; tokens/s normalised to the 16-head workload (token-heads/s / 16)')
    return dict(value=value, unit='tokens/s', cores=threads, kind='port', sample=sample)


def run_reference_arm(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    cb = cpu_baseline(seconds_budget=max(10.0, 8.0 * args.steps))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': cb['value'], 'unit': 'tokens/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': B * T / cb['value'] * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'chunk_gated_delta_rule fwd+bwd B4 T4096 H16 K=V=128 (CPU: bounded sample)'},
        'cpu_baseline': cb,
        'e2e': {'value': cb['value'], 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == 'reference':
        return run_reference_arm(args)

    import torch.distributed as dist
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    dev = torch.device('cuda', local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)

    import b200gdn
    from b200gdn import chunk_gated_delta_rule
    b200gdn.load_library()   # fails loudly when the CUDA library is missing
    peaks = load_peaks()

    host = make_batch(seed=rank, pin=True)
    batch = {n: x.to(dev) for n, x in host.items()}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step_device(batch, chunk_gated_delta_rule)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    stream = torch.cuda.current_stream(dev)
    launches0 = b200gdn.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step_device(batch, chunk_gated_delta_rule)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = b200gdn.launch_count() - launches0

    # end to end: every step copies its inputs from pinned host memory and all of its results (o and the five
    # gradients) back to pinned host memory.  The three legs run on three streams over three buffer slots, so the copy
    # of step i+1 and the read-back of step i-1 overlap the kernels of step i (PCIe is full duplex); a step's kernels
    # still wait for its own inputs and its read-back for its own results.
    NSLOT = 3
    out_host = [{n: torch.empty_like(host[n]).pin_memory() for n in ('q', 'k', 'v', 'g', 'beta')} for _ in range(NSLOT)]
    o_host = [torch.empty(B, T, HV, V, dtype=torch.bfloat16).pin_memory() for _ in range(NSLOT)]
    dev_in = [{n: torch.empty_like(x, device=dev) for n, x in host.items()} for _ in range(NSLOT)]
    h2d = sum(x.numel() * x.element_size() for x in host.values())
    d2h = sum(x.numel() * x.element_size() for x in out_host[0].values()) + o_host[0].numel() * 2
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def run_e2e(n_steps):
        """Returns device milliseconds from the first copy-in to the last copy-out."""
        torch.cuda.synchronize(dev)
        ev_in = [None] * n_steps
        ev_comp = [None] * n_steps
        ev_out = [None] * n_steps
        keep = [None] * NSLOT
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(s_in)
        for i in range(n_steps):
            slot = i % NSLOT
            if i >= NSLOT:
                s_in.wait_event(ev_comp[i - NSLOT])     # the slot's previous inputs have been consumed
                ev_out[i - NSLOT].synchronize()         # and its previous results are on the host: drop them
            with torch.cuda.stream(s_in):
                for n, x in host.items():
                    dev_in[slot][n].copy_(x, non_blocking=True)
                ev_in[i] = torch.cuda.Event()
                ev_in[i].record(s_in)
            stream.wait_event(ev_in[i])
            o, leaves = step_device(dev_in[slot], chunk_gated_delta_rule)
            ev_comp[i] = torch.cuda.Event()
            ev_comp[i].record(stream)
            keep[slot] = (o, leaves)                    # alive until the read-back below has finished
            s_out.wait_event(ev_comp[i])
            with torch.cuda.stream(s_out):
                o_host[slot].copy_(o, non_blocking=True)
                for n, leaf in zip(('q', 'k', 'v', 'g', 'beta'), leaves):
                    out_host[slot][n].copy_(leaf.grad, non_blocking=True)
                ev_out[i] = torch.cuda.Event()
                ev_out[i].record(s_out)
        t1.record(s_out)
        torch.cuda.synchronize(dev)
        return t0.elapsed_time(t1)
    run_e2e(3)
    barrier()
    ms_e2e = run_e2e(args.steps)
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    if world > 1:
        tt = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()

    if rank == 0:
        stages = time_stages(batch, min(args.steps, 10))
        tokens = B * T * world
        value = tokens * args.steps / (ms * 1e-3)
        e2e_value = tokens * args.steps / (ms_e2e * 1e-3)
        tok_heads = B * T * HV
        top = max(stages, key=lambda n: stages[n])
        n_chunks = B * (T // BT)
        sbytes = stage_bytes(B * T, n_chunks, B)
        per_stage = {}
        for n, t_ms in stages.items():
            gbs = sbytes[n] / (t_ms * 1e-3) / 1e9
            tfs = tok_heads * STAGE_FLOPS[n] / (t_ms * 1e-3) / 1e12
            per_stage[n] = {'ms': t_ms, 'GB/s': gbs, 'hbm_frac': gbs / peaks['hbm'], 'TFLOP/s': tfs,
                            'tensor_frac': tfs / peaks['bf16']}
        # every kernel of this path moves ~0.3-0.7 GB for 20-45 GFLOP: the HBM floor is 3-4x the tensor floor
        top_gbs = per_stage[top]['GB/s']
        step_tflops = tok_heads * (F_FWD + F_BWD) * args.steps / (ms * 1e-3) / 1e12
        line = {
            'metric': METRIC, 'value': value, 'unit': 'tokens/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms / args.steps, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {'workload': 'chunk_gated_delta_rule fwd+bwd B4 T4096 H16 HV16 K=V=128 chunk 64, fp32 h0, per GPU',
                       'l2': 'working set per step (>1 GiB) exceeds the 126 MB L2; no explicit flush',
                       'parallelism': f'dp{world} (batch/head shard, no collective)'},
            'pct_tensor_peak': 100.0 * step_tflops / world / peaks['bf16'],
            'step_tflops_per_gpu': step_tflops / world,
            'roofline': {'kernel': top, 'bound': 'hbm', 'achieved': top_gbs, 'peak': peaks['hbm'], 'unit': 'GB/s',
                         'frac': top_gbs / peaks['hbm'], 'traffic': NCU_TRAFFIC_BYTES.get(top),
                         'algorithmic_bytes': sbytes[top], 'peak_source': peaks['source'],
                         'step_hbm_frac': sum(sbytes.values()) / (sum(stages.values()) * 1e-3) / 1e9 / peaks['hbm'],
                         'stage_ms': stages, 'stages': per_stage},
            'e2e': {'value': e2e_value, 'unit': 'tokens/s', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
                    'ms_per_step': ms_e2e / args.steps,
                    'pipeline': 'copy-in, kernels and copy-out of consecutive steps overlap on three streams (3 buffer slots)'},
            'gpu_launches': launches,
            'clocks': clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line['cpu_baseline'] = cpu_baseline()
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == '__main__':
    main()

#!/usr/bin/env python
"""Benchmark of the chunked gated delta rule on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload train|fwd|varlen|heads|cp|decode|layer|modules]

Every run prints ONE JSON line.  The default workload (``train``) is the headline: one "step" is one forward +
backward pass of chunk_gated_delta_rule over one synthetic batch of B=4, T=4096, H=HV=16, K=V=128 (bf16 q/k/v,
fp32 g/beta, fp32 initial state): forward call + ``o.backward(do)``, the reference's own definition
(benchmarks/ops/run.py:246-255).  With N > 1 (launched by torch.distributed.run) every rank processes its own batch
of that shape (batch/head shard, no communication: weak scaling), the value is the sum over ranks divided by the
slowest rank's time, and the same line carries two sub-records that do exercise the multi-GPU design:
``heads_strong`` (B8 T8192 H32 split by heads over the ranks) and ``cp`` (one 524288-token sequence, context
parallel, checked against a single-GPU run before it is timed).

The other workloads time the remaining configurations of the specification through the same public API:
``fwd`` (forward only), ``varlen`` (16 packed sequences, 16 q/k + 32 value heads, forward + backward), ``heads``
(strong scaling by heads), ``cp`` (context parallel), ``decode`` (single-token steps, batch 1..256, state in place),
``layer`` (the headline shape called the way fla.layers.GatedDeltaNet calls the op), ``modules`` (the short convolution
and the gated RMS norm either side of the mixer).

``--impl reference`` times the reference's own naive recurrence (from a reference install under baseline/_ref when
there is one, else its restatement under oracle/) on a bounded sample of the headline workload on the host cores.
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
REF_INSTALL = os.path.join(ROOT, 'baseline', '_ref')
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)
if os.path.isdir(os.path.join(REF_INSTALL, 'fla')):
    sys.path.insert(0, REF_INSTALL)   # the reference install, when present, is the `fla` every leg of this script sees

import torch  # noqa: E402

METRIC = 'tokens/s chunk_gated_delta_rule fwd+bwd (B4 T4096 H16 D128 bf16); % tensor peak'
B, T, H, HV, K, V, BT = 4, 4096, 16, 16, 128, 128, 64

# algorithmic FLOPs per (token, value head), dense-tile counting, no recomputation
STAGE_FLOPS = {
    'intra_fwd': 2 * BT * (3 * K + V),                                 # K K^T, W, U | Q K^T
    'scan_out_fwd': 4 * K * V + 2 * K * V + 2 * BT * V,                # W S, K^T V~ | Q S, P V
    'scan_dvl_bwd': 6 * K * V + 2 * BT * (K + V),                      # K dS, Q^T do, W^T dv2 | P^T do (+ the Q K^T it does not redo)
    'bwd_dqk': 4 * K * V + 2 * BT * (V + 2 * K),                       # dP, do h^T, v dh^T, dP k, dP^T q
    'bwd_wy': 2 * K * V + 2 * BT * (5 * K + 2 * V + 2 * BT),           # dv2 h^T + WY backward
}
F_FWD = STAGE_FLOPS['intra_fwd'] + STAGE_FLOPS['scan_out_fwd']
F_BWD = STAGE_FLOPS['scan_dvl_bwd'] + STAGE_FLOPS['bwd_dqk'] + STAGE_FLOPS['bwd_wy']
assert F_FWD == 180224 and F_BWD == 409600


def algorithmic_bytes(R, Hq, Hv, NS, bwd=True):
    """Bytes a forward (+ backward) pass cannot avoid: every input read once, every result written once (plus the
    second read of q, k, v, g, beta by the backward pass); no intermediate counted."""
    qk, vv, vec, st = R * Hq * K * 2, R * Hv * V * 2, R * Hv * 4, NS * Hv * K * V * 4
    fwd = 2 * qk + vv + 2 * vec + st + vv + st                       # q k v g beta h0 -> o ht
    if not bwd:
        return fwd
    return fwd + 2 * qk + vv + 2 * vec + vv + st + 2 * qk + vv + 2 * vec + st   # re-read, do, dht -> dq dk dv dg dbeta dh0


def staged_bytes(R, C, NS):
    """HBM bytes of every kernel of one fwd+bwd step AS STAGED (each kernel's operands read once, its results written
    once, intermediates that pass between kernels through HBM included): what the kernels move, not the floor."""
    qk, wv = R * H * K * 2, R * HV * V * 2           # q or k ; v, u, v_new, do, dv2, o, dv
    w = R * HV * K * 2
    a_ = R * HV * BT * 2
    snap = C * HV * K * V * 2                         # h or dh snapshots
    st32 = NS * HV * K * V * 4                        # h0, ht, dht, dh0
    gam, vec = C * HV * BT * 4, R * HV * 4
    dkp = R * H * K * 2                               # chunk-local part of dk, bf16, passed through the dk buffer
    return {
        'intra_fwd': 2 * qk + wv + 2 * vec + 2 * a_ + w + wv + gam,                          # k q v -> A qk w u
        'scan_out_fwd': w + 2 * qk + wv + a_ + gam + st32 + snap + wv + st32 + wv,     # w k q u qk -> h v_new o
        'scan_dvl_bwd': 2 * qk + w + wv + a_ + gam + st32 + wv + snap + st32,          # q k w do qk -> dv2 dh dh0
        'bwd_dqk': 2 * qk + 2 * wv + 2 * snap + gam + qk + dkp + vec,
        'bwd_wy': qk + 2 * wv + a_ + snap + gam + 2 * vec + dkp + qk + wv + 2 * vec,
    }


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the headline workload from the ncu capture
# summarised in profiles/ (file and source revision below); a kernel missing here was not captured.  The constant goes
# stale with every kernel change: refresh it together with the profile.
NCU_TRAFFIC = {
    'source': 'profiles/chunk_fwd_bwd_B4_T4096_H16_D128_tcgen05.md',
    'kernel_sources_commit': 'fa829f3',
    'bytes': {'intra_fwd': 359.5e6, 'scan_out_fwd': 536.9e6, 'scan_dvl_bwd': 472.7e6, 'bwd_dqk': 650.1e6, 'bwd_wy': 549.8e6},
}


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


# --------------------------------------------------------------------------------------------- inputs
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


def device_inputs(Bn, Tn, Hn, HVn, dev, seed, h0_seqs=0, raw=False):
    """The same distributions generated on the device (the large configurations would take minutes on the host).
    ``raw``: q, k unnormalised and g, beta pre-activation, for the in-kernel options of the layer."""
    gen = torch.Generator(device=dev).manual_seed(seed)
    nrm = torch.nn.functional.normalize
    rn = lambda *s: torch.randn(*s, device=dev, generator=gen)
    q, k = rn(Bn, Tn, Hn, K), rn(Bn, Tn, Hn, K)
    if not raw:
        q, k = nrm(q, p=2, dim=-1), nrm(k, p=2, dim=-1)
    d = {'q': q.to(torch.bfloat16), 'k': k.to(torch.bfloat16), 'v': rn(Bn, Tn, HVn, V).to(torch.bfloat16)}
    g, beta = rn(Bn, Tn, HVn), rn(Bn, Tn, HVn)
    d['g'] = g if raw else torch.nn.functional.logsigmoid(g)
    d['beta'] = beta if raw else torch.sigmoid(beta)
    d['do'] = rn(Bn, Tn, HVn, V).to(torch.bfloat16)
    d['h0'] = rn(h0_seqs, HVn, K, V) * 0.1 if h0_seqs else None
    return d


def fwd_bwd(d, op, **kw):
    leaves = [d[n].detach().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
    o, ht = op(*leaves, initial_state=d.get('h0'), output_final_state=d.get('h0') is not None, **kw)
    o.backward(d['do'])
    return o, leaves


def timed(fn, steps, warmup, dev, barrier):
    """Device milliseconds of `steps` calls of fn (CUDA events on the current stream, barriers on both sides)."""
    for _ in range(warmup):
        fn()
    barrier()
    stream = torch.cuda.current_stream(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    barrier()
    return e0.elapsed_time(e1)


def err_ratio(ref, out):
    ref, out = ref.detach().float(), out.detach().float()
    return float((ref - out).square().mean().sqrt() / (ref.square().mean().sqrt() + 1e-12))


# --------------------------------------------------------------------------------------------- per-kernel timing
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
               A=torch.empty(rows, HV, 64, **bf), qk=torch.empty(rows, HV, 64, **bf), w=torch.empty(rows, HV, K, **bf),
               u=torch.empty(rows, HV, V, **bf),
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
    plan = [('intra_fwd', 'b200gdn_chunk_fwd', _lib.FWD_INTRA), ('scan_out_fwd', 'b200gdn_chunk_fwd', _lib.FWD_SCAN | _lib.FWD_OUT),
            ('scan_dvl_bwd', 'b200gdn_chunk_bwd', _lib.BWD_DVLOCAL | _lib.BWD_SCAN), ('bwd_dqk', 'b200gdn_chunk_bwd', _lib.BWD_DQKWG),
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


# --------------------------------------------------------------------------------------------- CPU legs
def _naive_reference():
    """The naive recurrence to time on the host: the reference's own function when a reference install is importable
    (kind "reference"), else its restatement under oracle/ (kind "port").  Both take (q, k, v, beta, g, ...) /
    (q, k, v, g, beta, ...) in their own order; returns (callable(q,k,v,g,beta,scale,h0) -> (o, ht), kind)."""
    try:
        from fla.ops.gated_delta_rule.naive import naive_recurrent_gated_delta_rule as ref_fn

        def call(q, k, v, g, beta, scale, h0):
            return ref_fn(q=q, k=k, v=v, beta=beta, g=g, scale=scale, initial_state=h0, output_final_state=True)
        return call, 'reference'
    except Exception:
        from oracle.gdn_oracle import naive_recurrent

        def call(q, k, v, g, beta, scale, h0):
            return naive_recurrent(q, k, v, g, beta, scale=scale, initial_state=h0, output_final_state=True)
        return call, 'port'


def cpu_baseline(seconds_budget=20.0, threads=None):
    """The naive recurrence on the host cores.  (1) A bounded sample of the headline workload: forward + backward by
    autograd on B1 T1024 H4 K=V=128 (same distributions), tokens/s normalised to the 16-head workload.  (2) The
    specification's first configuration exactly: B1 T1024 H4 K=V=64 fp32, forward only, final state on, with all
    host threads and with one thread, tokens/s = 1024 / t (median of 5 runs after one warm-up)."""
    from oracle.gdn_oracle import make_inputs
    call, kind = _naive_reference()
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    Bs, Ts, Hs = 1, 1024, 4
    d = make_inputs(Bs, Ts, Hs, Hs, K, V, seed=0)

    def one():
        leaves = [d[n].clone().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
        o, ht = call(*leaves, K ** -0.5, d['h0'])
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
    value = (Bs * Ts * Hs / HV) / t   # tokens/s of the full 16-head workload = token-heads per second / 16

    c1 = make_inputs(1, 1024, 4, 4, 64, 64, seed=0, h0_std=0.0)

    def config1():
        with torch.no_grad():
            call(c1['q'], c1['k'], c1['v'], c1['g'], c1['beta'], 64 ** -0.5, torch.zeros_like(c1['h0']))

    def median5():
        config1()
        ts = []
        for _ in range(5):
            t0 = time.perf_counter()
            config1()
            ts.append(time.perf_counter() - t0)
        return statistics.median(ts)
    t_all = median5()
    torch.set_num_threads(1)
    t_one = median5()
    torch.set_num_threads(threads)
    sample = (f'naive recurrence fwd+bwd (autograd), B={Bs} T={Ts} H=HV={Hs} K=V={K} fp32, median of {max(reps, 1)} runs of '
              f'{t:.2f} s; tokens/s normalised to the 16-head workload (token-heads/s / 16)')
    return dict(value=value, unit='tokens/s', cores=threads, kind=kind, sample=sample,
                config1={'workload': 'naive recurrence forward, B1 T1024 H4 K=V=64 fp32, zero initial state, final state on',
                         'tokens_per_s': 1024 / t_all, 'threads': threads, 'tokens_per_s_1_thread': 1024 / t_one,
                         'seconds': t_all, 'seconds_1_thread': t_one})


def run_reference_arm(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    cb = cpu_baseline(seconds_budget=max(10.0, 8.0 * args.steps))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': cb['value'], 'unit': 'tokens/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': B * T / cb['value'] * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'chunk_gated_delta_rule fwd+bwd B4 T4096 H16 K=V=128 (CPU: the naive recurrence on a bounded '
                               'sample, extrapolated by token-heads)'},
        'cpu_baseline': cb,
        'e2e': {'value': cb['value'], 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------- GPU baseline (worker)
def gpu_baseline_worker():
    """Child process: the reference's stock Triton chunk_gated_delta_rule (dispatch to other back ends disabled) from
    the install under baseline/_ref, on the headline tensors, timed with CUDA events next to this library's path in
    the same process; prints one JSON object.  Informational: the `--impl reference` arm stays the CPU recurrence."""
    os.environ['FLA_DISABLE_BACKEND_DISPATCH'] = '1'
    import fla
    from fla.ops.gated_delta_rule import chunk_gated_delta_rule as ref_op
    from b200gdn import chunk_gated_delta_rule as our_op
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    d = make_batch(seed=0, device=dev)

    def run(op):
        leaves = [d[n].detach().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
        h0 = d['h0'].detach().requires_grad_(True)
        o, ht = op(*leaves, initial_state=h0, output_final_state=True)
        o.backward(d['do'])
        return [o, ht] + [x.grad for x in leaves] + [h0.grad]

    def clock(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n
    out = {'fla_version': fla.__version__}
    for _ in range(5):   # autotuning and warm-up
        ref = run(ref_op)
    for _ in range(5):
        ours = run(our_op)
    out['ref_fwd_bwd_ms'] = clock(lambda: run(ref_op), 20)
    out['ours_fwd_bwd_ms'] = clock(lambda: run(our_op), 20)
    with torch.no_grad():
        f_ref = lambda: ref_op(d['q'], d['k'], d['v'], d['g'], d['beta'], initial_state=d['h0'], output_final_state=True)
        f_our = lambda: our_op(d['q'], d['k'], d['v'], d['g'], d['beta'], initial_state=d['h0'], output_final_state=True)
        for _ in range(3):
            f_ref(), f_our()
        out['ref_fwd_ms'] = clock(f_ref, 20)
        out['ours_fwd_ms'] = clock(f_our, 20)
    names = ('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta', 'dh0')
    out['err_ratio_vs_reference'] = {n: err_ratio(r, x) for n, r, x in zip(names, ref, ours)}
    out['speedup_fwd_bwd'] = out['ref_fwd_bwd_ms'] / out['ours_fwd_bwd_ms']
    out['speedup_fwd'] = out['ref_fwd_ms'] / out['ours_fwd_ms']
    print('GPU_BASELINE ' + json.dumps(out))


def gpu_baseline(timeout=420):
    if not os.path.isdir(os.path.join(REF_INSTALL, 'fla')):
        return None
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), '--worker', 'gpu_baseline'], capture_output=True,
                           text=True, timeout=timeout)
        for ln in r.stdout.splitlines():
            if ln.startswith('GPU_BASELINE '):
                return json.loads(ln[len('GPU_BASELINE '):])
        return {'unavailable': (r.stderr or r.stdout)[-300:]}
    except Exception as e:  # informational field: never fails the bench
        return {'unavailable': repr(e)[:300]}


# --------------------------------------------------------------------------------------------- distributed plumbing
class Dist:
    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get('WORLD_SIZE', '1'))
        self.rank = int(os.environ.get('RANK', '0'))
        self.local_rank = int(os.environ.get('LOCAL_RANK', '0'))
        self.dev = torch.device('cuda', self.local_rank)
        torch.cuda.set_device(self.dev)
        if self.world > 1:
            dist.init_process_group('nccl', device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, *vals):
        if self.world == 1:
            return list(vals)
        t = torch.tensor(vals, device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def base_line(args, D, metric, value, ms_per_step, scaling, workload, **config):
    return {'metric': metric, 'value': value, 'unit': 'tokens/s', 'n_gpus': D.world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': scaling, 'vs_baseline': None, 'dtype': 'bf16',
            'data': 'synthetic', 'config': dict(workload=workload, **config)}


def tensor_roofline(kernel, flops, ms, peaks, traffic=None):
    tf = flops / (ms * 1e-3) / 1e12
    return {'kernel': kernel, 'bound': 'tensor', 'achieved': tf, 'peak': peaks['bf16'], 'unit': 'TFLOP/s', 'frac': tf / peaks['bf16'],
            'frac_of_sustained': tf / peaks['bf16_sustained'], 'peak_source': peaks['source'], 'traffic': traffic}


# --------------------------------------------------------------------------------------------- workloads
def heads_strong(args, D, steps, warmup, with_single=True):
    """B8 T8192 H32 K=V=128 forward + backward split by heads over the ranks (rank r takes heads [r 32/W, (r+1) 32/W)),
    no communication; global tokens/s.  On rank 0 the whole problem is also timed on one GPU so that the strong-scaling
    efficiency can be read off."""
    from b200gdn import chunk_gated_delta_rule
    Bn, Tn, Hn = 8, 8192, 32
    hs = Hn // D.world
    d = device_inputs(Bn, Tn, hs, hs, D.dev, seed=100 + D.rank)
    ms = timed(lambda: fwd_bwd(d, chunk_gated_delta_rule), steps, warmup, D.dev, D.barrier)
    (ms,) = D.max_over_ranks(ms)
    del d
    single = None
    if with_single and D.world > 1:
        if D.rank == 0:
            d = device_inputs(Bn, Tn, Hn, Hn, D.dev, seed=100)
            single = timed(lambda: fwd_bwd(d, chunk_gated_delta_rule), steps, warmup, D.dev, lambda: torch.cuda.synchronize(D.dev)) / steps
            del d
        D.barrier()
    torch.cuda.empty_cache()
    rec = {'workload': f'B{Bn} T{Tn} H{Hn} K=V=128 fwd+bwd, {hs} heads per rank, no collective', 'tokens_per_s': Bn * Tn * steps / (ms * 1e-3),
           'ms_per_step': ms / steps, 'scaling': 'strong'}
    if single is not None:
        rec['single_gpu_ms_per_step'] = single
        rec['strong_scaling_efficiency'] = single / (ms / steps) / D.world
    return rec


def context_parallel(args, D, steps, warmup, Tn=524288):
    """One sequence of 524288 tokens (H16 K=V=128), forward + backward, split into equal contiguous shards over the
    ranks (fla/ops/cp semantics).  Before timing, every rank runs the whole sequence on its own GPU and compares its
    shard of o, dq, dk, dv, dg, dbeta with the context-parallel result; a failed check ends the bench non-zero."""
    import b200gdn.cp as cp
    from b200gdn import build_cp_context, chunk_gated_delta_rule
    Hn = 16
    W, r = D.world, D.rank
    full = device_inputs(1, Tn, Hn, Hn, D.dev, seed=7)
    part = Tn // W
    sl = slice(r * part, (r + 1) * part)
    shard = {n: (x[:, sl].contiguous() if x is not None else None) for n, x in full.items()}
    o, leaves = fwd_bwd(full, chunk_gated_delta_rule)
    want = [o[:, sl].clone()] + [x.grad[:, sl].clone() for x in leaves]
    single_ms = None
    if r == 0:
        single_ms = timed(lambda: fwd_bwd(full, chunk_gated_delta_rule), max(2, steps // 4), 1, D.dev,
                          lambda: torch.cuda.synchronize(D.dev)) / max(2, steps // 4)
    del o, leaves, full
    torch.cuda.empty_cache()
    if W == 1:
        rec = {'workload': f'B1 T{Tn} H{Hn} K=V=128 fwd+bwd, single GPU (context parallelism needs 2 or more ranks)',
               'tokens_per_s': Tn / (single_ms * 1e-3), 'ms_per_step': single_ms}
        return rec, True
    cu = torch.tensor([0, Tn], dtype=torch.int32, device=D.dev)
    ctx = build_cp_context(cu, group=D.dist.group.WORLD, cu_seqlens_cpu=torch.tensor([0, Tn], dtype=torch.int32))
    o, leaves = fwd_bwd(shard, chunk_gated_delta_rule, cp_context=ctx)
    got = [o] + [x.grad for x in leaves]
    names = ('o', 'dq', 'dk', 'dv', 'dg', 'dbeta')
    errs = [err_ratio(wv, gv) for wv, gv in zip(want, got)]
    errs = D.max_over_ranks(*errs)
    tol = dict(o=0.005, dq=0.008, dk=0.008, dv=0.008, dg=0.02, dbeta=0.02)
    ok = all(e <= tol[n] for n, e in zip(names, errs))
    del o, leaves, got, want
    cp.PHASE_TIMES = {}
    ms = timed(lambda: fwd_bwd(shard, chunk_gated_delta_rule, cp_context=ctx), steps, warmup, D.dev, D.barrier)
    phases = cp.collect_phase_times() if hasattr(cp, 'collect_phase_times') else None
    cp.PHASE_TIMES = None
    (ms,) = D.max_over_ranks(ms)
    (single_ms,) = D.max_over_ranks(single_ms or 0.0)
    rec = {'workload': f'B1 T{Tn} H{Hn} K=V=128 fwd+bwd, {W} equal contiguous shards of {part} tokens',
           'tokens_per_s': Tn * steps / (ms * 1e-3), 'ms_per_step': ms / steps, 'single_gpu_ms_per_step': single_ms,
           'scaling_efficiency': single_ms / (ms / steps) / W, 'exchange_bytes_per_rank_per_direction': Hn * K * (K + V) * 4,
           'parity_vs_single_gpu': dict(zip(names, errs)), 'parity_ok': ok, 'phases_ms_rank0': phases}
    return rec, ok


def workload_train(args, D):
    import b200gdn
    from b200gdn import chunk_gated_delta_rule
    peaks = load_peaks()
    dev, world, rank = D.dev, D.world, D.rank
    host = make_batch(seed=rank, pin=True)
    batch = {n: x.to(dev) for n, x in host.items()}
    step = lambda: fwd_bwd(batch, chunk_gated_delta_rule)

    for _ in range(args.warmup):
        step()
    D.barrier()
    sampler = ClockSampler(D.local_rank)
    if rank == 0:
        sampler.start()
    stream = torch.cuda.current_stream(dev)
    launches0 = b200gdn.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    D.barrier()
    t_host0 = time.perf_counter()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    host_us = (time.perf_counter() - t_host0) / args.steps * 1e6   # enqueue time of one step (launches run behind it)
    D.barrier()
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
        ev_in, ev_comp, ev_out = [None] * n_steps, [None] * n_steps, [None] * n_steps
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
            o, leaves = fwd_bwd(dev_in[slot], chunk_gated_delta_rule)
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
    D.barrier()
    ms_e2e = run_e2e(args.steps)
    D.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms, ms_e2e, host_us = D.max_over_ranks(ms, ms_e2e, host_us)

    stages = time_stages(batch, min(args.steps, 10)) if rank == 0 else None
    del batch, dev_in, out_host, o_host
    torch.cuda.empty_cache()
    sub = {}
    if world > 1:
        sub['heads_strong'] = heads_strong(args, D, max(3, args.steps // 4), 2)
        rec, ok = context_parallel(args, D, max(3, args.steps // 4), 2)
        sub['cp'] = rec
        if not ok:
            if rank == 0:
                print(json.dumps({'error': 'context-parallel result differs from the single-GPU result', 'cp': rec}), file=sys.stderr)
            D.close()
            sys.exit(3)

    if rank == 0:
        tokens = B * T * world
        value = tokens * args.steps / (ms * 1e-3)
        e2e_value = tokens * args.steps / (ms_e2e * 1e-3)
        tok_heads = B * T * HV
        top = max(stages, key=lambda n: stages[n])
        sb = staged_bytes(B * T, B * (T // BT), B)
        alg = algorithmic_bytes(B * T, H, HV, B)
        per_stage = {}
        for n, t_ms in stages.items():
            gbs = sb[n] / (t_ms * 1e-3) / 1e9
            tfs = tok_heads * STAGE_FLOPS[n] / (t_ms * 1e-3) / 1e12
            per_stage[n] = {'ms': t_ms, 'staged_MB': sb[n] / 1e6, 'GB/s_of_staged_bytes': gbs, 'hbm_frac_of_staged_bytes': gbs / peaks['hbm'],
                            'TFLOP/s': tfs, 'tensor_frac': tfs / peaks['bf16']}
        step_ms = ms / args.steps
        step_tflops = tok_heads * (F_FWD + F_BWD) / (step_ms * 1e-3) / 1e12
        roof = tensor_roofline(top, tok_heads * STAGE_FLOPS[top], stages[top], peaks, NCU_TRAFFIC['bytes'].get(top))
        roof.update({
            'traffic_source': NCU_TRAFFIC['source'], 'traffic_kernel_sources_commit': NCU_TRAFFIC['kernel_sources_commit'],
            'step': {'TFLOP/s': step_tflops, 'frac': step_tflops / peaks['bf16'], 'frac_of_sustained': step_tflops / peaks['bf16_sustained'],
                     'algorithmic_bytes_step': alg, 'staged_bytes_step': sum(sb.values()), 'staged_over_algorithmic': sum(sb.values()) / alg,
                     'traffic_step': sum(NCU_TRAFFIC['bytes'].values()), 'traffic_over_algorithmic': sum(NCU_TRAFFIC['bytes'].values()) / alg,
                     'GB/s_of_algorithmic_bytes': alg / (step_ms * 1e-3) / 1e9,
                     'hbm_frac_of_algorithmic_bytes': alg / (step_ms * 1e-3) / 1e9 / peaks['hbm'],
                     'hbm_frac_of_staged_bytes': sum(sb.values()) / (sum(stages.values()) * 1e-3) / 1e9 / peaks['hbm'],
                     'hbm_peak_GB/s': peaks['hbm']},
            'stage_ms': stages, 'stages': per_stage})
        line = base_line(args, D, METRIC, value, step_ms, 'weak',
                         'chunk_gated_delta_rule fwd+bwd B4 T4096 H16 HV16 K=V=128 chunk 64, fp32 h0, per GPU',
                         l2='working set per step (>1 GiB) exceeds the 126 MB L2; no explicit flush',
                         parallelism=f'dp{world} (batch/head shard, no collective)')
        line.update({
            'pct_tensor_peak': 100.0 * step_tflops / peaks['bf16'], 'step_tflops_per_gpu': step_tflops,
            'roofline': roof,
            'e2e': {'value': e2e_value, 'unit': 'tokens/s', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
                    'ms_per_step': ms_e2e / args.steps, 'h2d_GB/s': h2d / (ms_e2e / args.steps * 1e-3) / 1e9,
                    'd2h_GB/s': d2h / (ms_e2e / args.steps * 1e-3) / 1e9,
                    'pipeline': 'copy-in, kernels and copy-out of consecutive steps overlap on three streams (3 buffer slots)'},
            'gpu_launches': launches, 'host_us_per_step': host_us, 'clocks': clocks})
        line.update(sub)
        if world == 1 and not args.no_cpu_baseline:
            line['cpu_baseline'] = cpu_baseline()
        if world == 1:
            line['gpu_baseline'] = None if args.no_gpu_baseline else gpu_baseline()
        print(json.dumps(line))


def workload_simple(args, D, name):
    """fwd / varlen / layer: one configuration per rank (weak scaling when N > 1), through the public API."""
    import b200gdn
    from b200gdn import chunk_gated_delta_rule
    from oracle.gdn_oracle import random_cu_seqlens
    peaks = load_peaks()
    dev = D.dev
    extra = {}
    if name == 'fwd':
        d = device_inputs(B, T, H, HV, dev, seed=D.rank, h0_seqs=B)

        def step():
            with torch.no_grad():
                chunk_gated_delta_rule(d['q'], d['k'], d['v'], d['g'], d['beta'], initial_state=d['h0'], output_final_state=True)
        tokens, heads, flops = B * T, HV, F_FWD
        metric = 'tokens/s chunk_gated_delta_rule forward (B4 T4096 H16 D128 bf16)'
        wl = 'chunk_gated_delta_rule forward B4 T4096 H16 HV16 K=V=128, fp32 h0, final state on'
        abytes = algorithmic_bytes(B * T, H, HV, B, bwd=False)
    elif name == 'varlen':
        cu = random_cu_seqlens(16, 65536, 256, 8192, seed=0)
        d = device_inputs(1, 65536, 16, 32, dev, seed=D.rank, h0_seqs=16)
        cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
        cu_c = torch.tensor(cu, dtype=torch.int32)

        def step():
            leaves = [d[n].detach().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
            h0 = d['h0'].detach().requires_grad_(True)
            o, ht = chunk_gated_delta_rule(*leaves, initial_state=h0, output_final_state=True, cu_seqlens=cu_t, cu_seqlens_cpu=cu_c)
            o.backward(d['do'])
        tokens, heads, flops = 65536, 32, F_FWD + F_BWD
        metric = 'tokens/s chunk_gated_delta_rule fwd+bwd (16 packed sequences, 65536 tokens, H16 HV32 D128 bf16)'
        wl = 'chunk_gated_delta_rule fwd+bwd, 16 sequences packed by cu_seqlens (lengths in [256, 8192], 65536 tokens), H16 HV32 K=V=128, fp32 h0'
        extra['cu_seqlens'] = cu
        abytes = algorithmic_bytes(65536, 16, 32, 16)
    else:   # layer
        d = device_inputs(B, T, H, HV, dev, seed=D.rank, h0_seqs=B, raw=True)
        A_log = torch.log(torch.empty(HV, device=dev).uniform_(1, 16))
        dt_bias = torch.randn(HV, device=dev) * 0.1
        h0 = d['h0'].transpose(-1, -2).contiguous()

        def step():
            leaves = [d[n].detach().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
            o, ht = chunk_gated_delta_rule(*leaves, initial_state=h0, output_final_state=True, use_qk_l2norm_in_kernel=True,
                                           use_gate_in_kernel=True, A_log=A_log, dt_bias=dt_bias, use_beta_sigmoid_in_kernel=True,
                                           state_v_first=True)
            o.backward(d['do'])
        tokens, heads, flops = B * T, HV, F_FWD + F_BWD
        metric = 'tokens/s chunk_gated_delta_rule fwd+bwd with the layer\'s in-kernel options (B4 T4096 H16 D128 bf16)'
        wl = ('chunk_gated_delta_rule fwd+bwd B4 T4096 H16 K=V=128 as fla.layers.GatedDeltaNet calls it: q/k L2 norm, '
              'gate -exp(A_log) softplus(g + dt_bias), sigmoid beta, V-first state')
        abytes = algorithmic_bytes(B * T, H, HV, B)
    launches0 = b200gdn.launch_count()
    ms = timed(step, args.steps, args.warmup, dev, D.barrier)
    launches = (b200gdn.launch_count() - launches0) * args.steps // (args.steps + args.warmup)
    (ms,) = D.max_over_ranks(ms)
    if D.rank == 0:
        step_ms = ms / args.steps
        line = base_line(args, D, metric, tokens * D.world * args.steps / (ms * 1e-3), step_ms, 'weak', wl,
                         parallelism=f'dp{D.world} (one configuration per rank, no collective)', **extra)
        roof = tensor_roofline('whole step', tokens * heads * flops, step_ms, peaks)
        roof['algorithmic_bytes_step'] = abytes
        roof['hbm_frac_of_algorithmic_bytes'] = abytes / (step_ms * 1e-3) / 1e9 / peaks['hbm']
        line.update({'roofline': roof, 'gpu_launches': launches})
        print(json.dumps(line))


def workload_heads(args, D):
    rec = heads_strong(args, D, args.steps, args.warmup)
    if D.rank == 0:
        peaks = load_peaks()
        line = base_line(args, D, 'tokens/s chunk_gated_delta_rule fwd+bwd (B8 T8192 H32 D128 bf16), heads split over the GPUs',
                         rec['tokens_per_s'], rec['ms_per_step'], 'strong', rec['workload'], parallelism=f'heads over {D.world} GPUs, no collective')
        line['roofline'] = tensor_roofline('whole step', 8 * 8192 * 32 / D.world * (F_FWD + F_BWD), rec['ms_per_step'], peaks)
        line['heads_strong'] = rec
        print(json.dumps(line))


def workload_cp(args, D):
    rec, ok = context_parallel(args, D, args.steps, args.warmup)
    if D.rank == 0:
        peaks = load_peaks()
        line = base_line(args, D, 'tokens/s chunk_gated_delta_rule fwd+bwd (B1 T524288 H16 D128 bf16), context parallel',
                         rec['tokens_per_s'], rec['ms_per_step'], 'strong', rec['workload'],
                         parallelism=f'sequence over {D.world} GPUs, one all-gather of (M, h) pairs per direction')
        line['roofline'] = tensor_roofline('whole step', 524288 * 16 / D.world * (F_FWD + F_BWD), rec['ms_per_step'], peaks)
        line['cp'] = rec
        print(json.dumps(line))
    if not ok:
        D.close()
        sys.exit(3)


def workload_decode(args, D):
    """Single-token steps of fused_recurrent_gated_delta_rule, batch 1..256, [B,16,128,128] fp32 state updated in place.
    The states live in a pool larger than L2 and every step addresses another set of slots, so each step really moves
    its 2 * B MiB through HBM; a CUDA graph of one pass over the pool is replayed, so the figure is kernel time."""
    from b200gdn import fused_recurrent_gated_delta_rule
    peaks = load_peaks()
    dev = D.dev
    Hn = 16
    table = []
    for Bn in args.decode_batches:
        n_sets = max(2, 512 // Bn)                      # pool of at least 512 MiB: four times L2
        pool = torch.randn(n_sets * Bn, Hn, K, V, device=dev) * 0.1
        d = device_inputs(Bn, 1, Hn, Hn, dev, seed=Bn)
        idx = [torch.arange(i * Bn, (i + 1) * Bn, device=dev, dtype=torch.int32) for i in range(n_sets)]

        def one_pass():
            for i in range(n_sets):
                fused_recurrent_gated_delta_rule(d['q'], d['k'], d['v'], d['g'], beta=d['beta'], initial_state=pool,
                                                 output_final_state=True, state_indices=idx[i])
        one_pass()
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_pass()
        for _ in range(max(3, args.warmup)):
            graph.replay()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(2, args.steps // 2)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        us = e0.elapsed_time(e1) * 1e3 / (reps * n_sets)
        nbytes = 2 * Bn * Hn * K * V * 4
        table.append({'batch': Bn, 'us_per_step': us, 'steps_per_s': 1e6 / us, 'GB/s': nbytes / us / 1e3,
                      'hbm_frac': nbytes / us / 1e3 / peaks['hbm']})
        del pool, graph
        torch.cuda.empty_cache()
    if D.rank == 0:
        top = table[-1]
        line = base_line(args, D, 'decode steps/s of fused_recurrent_gated_delta_rule (one token per sequence, [B,16,128,128] fp32 state in place)',
                         top['steps_per_s'], top['us_per_step'] / 1e3, 'weak', 'decode sweep B = ' + ','.join(str(b) for b in args.decode_batches) + ', H=HV=16 K=V=128, bf16 q/k/v, state pool of >= 512 MiB addressed by state_indices',
                         parallelism='replicas only', timing='CUDA graph of one pass over the pool, CUDA events around the replays')
        line['unit'] = f"steps/s (batch {top['batch']})"
        line['dtype'] = 'f32'
        line['roofline'] = {'kernel': 'decode_stream_kernel', 'bound': 'hbm', 'achieved': top['GB/s'], 'peak': peaks['hbm'], 'unit': 'GB/s',
                            'frac': top['hbm_frac'], 'traffic': None, 'peak_source': peaks['source'],
                            'algorithmic_bytes_per_step': '2 * B * 16 * 128 * 128 * 4'}
        line['sweep'] = table
        line['gpu_launches'] = sum(max(2, 512 // t['batch']) for t in table)
        print(json.dumps(line))


def workload_modules(args, D):
    """The two steps either side of the mixer at the headline shape, forward + backward each: the short causal convolution
    (kernel 4, SiLU) over the q / k / v projections [4, 4096, 2048] and the gated RMS norm over [4, 4096, 16, 128]; both
    are HBM streaming, reported as bytes moved (every tensor once per pass) over device time."""
    from b200gdn.modules import causal_conv1d, rms_norm_gated
    peaks = load_peaks()
    dev = D.dev
    gen = torch.Generator(device=dev).manual_seed(3)
    Dc, Wc = H * K, 4
    x = torch.randn(B, T, Dc, device=dev, generator=gen).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(Dc, Wc, device=dev, generator=gen) * 0.5).requires_grad_(True)
    bias = torch.randn(Dc, device=dev, generator=gen).requires_grad_(True)
    dy = torch.randn(B, T, Dc, device=dev, generator=gen).to(torch.bfloat16)

    def conv_step():
        y, _ = causal_conv1d(x, w, bias, activation='silu')
        torch.autograd.grad(y, (x, w, bias), dy)   # no accumulation into .grad: the step is the two kernels, nothing else
    o = torch.randn(B, T, HV, V, device=dev, generator=gen).to(torch.bfloat16).requires_grad_(True)
    gate = torch.randn(B, T, HV, V, device=dev, generator=gen).to(torch.bfloat16).requires_grad_(True)
    nw = torch.ones(V, device=dev, requires_grad=True)
    do = torch.randn(B, T, HV, V, device=dev, generator=gen).to(torch.bfloat16)

    def norm_step():
        torch.autograd.grad(rms_norm_gated(o, gate, nw, eps=1e-5), (o, gate, nw), do)
    def graph_ms(fn):
        """Device time of one step: the step is captured into a CUDA graph once and replayed, so that the figure is the
        kernels' time and not the host's launch path (three launches per step are shorter than their Python calls)."""
        fn()
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return timed(graph.replay, args.steps, args.warmup, dev, D.barrier) / args.steps
    ms_conv_eager = timed(conv_step, args.steps, args.warmup, dev, D.barrier) / args.steps
    ms_norm_eager = timed(norm_step, args.steps, args.warmup, dev, D.barrier) / args.steps
    timing = 'CUDA graph of one forward + backward, CUDA events around the replays; eager figures beside'
    try:
        ms_conv, ms_norm = graph_ms(conv_step), graph_ms(norm_step)
    except RuntimeError as e:   # a step that cannot be captured: the eager figures stand in, and the line says so
        ms_conv, ms_norm, timing = ms_conv_eager, ms_norm_eager, f'eager (graph capture failed: {str(e)[:80]})'
    nb = B * T * Dc * 2
    conv_bytes = 2 * nb + 3 * nb + (B * T // 32) * Dc * (Wc + 1) * 4 * 2   # x -> y ; x, dy -> dx ; parameter partials
    norm_bytes = 3 * nb + 5 * nb                                             # x, g -> y ; x, g, dy -> dx, dg
    if D.rank == 0:
        line = base_line(args, D, 'tokens/s of the short convolution + gated RMS norm around the mixer, fwd+bwd (B4 T4096 H16 D128 bf16)',
                         B * T / ((ms_conv * 3 + ms_norm) * 1e-3), ms_conv * 3 + ms_norm, 'weak',
                         'causal_conv1d (W=4, SiLU, bias) on q, k, v [4,4096,2048] each and rms_norm_gated on [4,4096,16,128], forward + backward',
                         parallelism='single GPU', timing=timing)
        line['roofline'] = {'kernel': 'conv_fwd + conv_bwd', 'bound': 'hbm', 'achieved': conv_bytes / (ms_conv * 1e-3) / 1e9, 'peak': peaks['hbm'],
                            'unit': 'GB/s', 'frac': conv_bytes / (ms_conv * 1e-3) / 1e9 / peaks['hbm'], 'traffic': None, 'peak_source': peaks['source']}
        line['modules'] = {'conv_fwd_bwd_ms': ms_conv, 'conv_GB/s': conv_bytes / (ms_conv * 1e-3) / 1e9,
                           'conv_hbm_frac': conv_bytes / (ms_conv * 1e-3) / 1e9 / peaks['hbm'],
                           'norm_gate_fwd_bwd_ms': ms_norm, 'norm_gate_GB/s': norm_bytes / (ms_norm * 1e-3) / 1e9,
                           'norm_gate_hbm_frac': norm_bytes / (ms_norm * 1e-3) / 1e9 / peaks['hbm'],
                           'eager_conv_fwd_bwd_ms': ms_conv_eager, 'eager_norm_gate_fwd_bwd_ms': ms_norm_eager}
        line['gpu_launches'] = 6 * (args.steps + args.warmup) * 2
        print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='train', choices=['train', 'fwd', 'varlen', 'heads', 'cp', 'decode', 'layer', 'modules'])
    ap.add_argument('--decode-batches', type=lambda t: [int(x) for x in t.split(',')], default=[1, 2, 4, 8, 16, 32, 64, 128, 256],
                    help='batch sizes of the decode sweep (the last one is the headline of that workload)')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-gpu-baseline', action='store_true')
    ap.add_argument('--worker', default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.worker == 'gpu_baseline':
        return gpu_baseline_worker()
    if args.impl == 'reference':
        return run_reference_arm(args)

    D = Dist()
    import b200gdn
    b200gdn.load_library()   # fails loudly when the CUDA library is missing
    if args.workload == 'train':
        workload_train(args, D)
    elif args.workload in ('fwd', 'varlen', 'layer'):
        workload_simple(args, D, args.workload)
    elif args.workload == 'heads':
        workload_heads(args, D)
    elif args.workload == 'cp':
        workload_cp(args, D)
    elif args.workload == 'modules':
        workload_modules(args, D)
    else:
        workload_decode(args, D)
    D.close()


if __name__ == '__main__':
    main()

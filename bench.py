#!/usr/bin/env python
"""Benchmark of the deformable-convolution forward (DCNv2) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c5|c2|c3] [--batch B]

One step = one forward over one batch of synthetic input.  The default workload is the
large-batch DCNv2 layer (N=256, C_in=C_out=256, 128x128, 3x3, deform_groups=8, bias,
bf16); with G GPUs the batch is split into G contiguous shards (strong scaling, no
collective on the data path).  Prints one JSON line on rank 0.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: N, C, H, W, Co, k, stride, pad, dil, groups, dg, offset sigma, mask, bias, int_frac, mask sigma
    'c1': dict(N=2, C=64, H=56, W=56, Co=64, k=3, s=1, p=1, d=1, g=1, dg=1, sigma=2.0,
               mask=True, bias=True, int_frac=0.0, msigma=1.0,
               desc='DCNv2 N=2 C=64 56x56 3x3 s1 p1 dg=1 bias'),
    'c5': dict(N=256, C=256, H=128, W=128, Co=256, k=3, s=1, p=1, d=1, g=1, dg=8, sigma=2.0,
               mask=True, bias=True, int_frac=0.0, msigma=1.0,
               desc='DCNv2 N=256 C=256 128x128 3x3 s1 p1 dg=8 bias'),
    'c2': dict(N=8, C=256, H=100, W=168, Co=256, k=3, s=1, p=1, d=1, g=1, dg=1, sigma=1.5,
               mask=False, bias=False, int_frac=0.0, msigma=1.0,
               desc='DCNv1 N=8 C=256 100x168 3x3 s1 p1 dg=1'),
    'c3': dict(N=4, C=512, H=64, W=64, Co=512, k=3, s=2, p=2, d=2, g=1, dg=4, sigma=8.0,
               mask=True, bias=True, int_frac=0.05, msigma=2.0,
               desc='DCNv2 N=4 C=512 64x64 3x3 s2 p2 d2 dg=4 bias'),
}

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the main kernel per sample, from
# an ncu capture of dcn_fwd_tc2 at batch 16 (253.3 MB read + 104.3 MB written = 357.6 MB); the
# traffic grows in proportion to the samples processed.  None where no capture exists.
NCU_TRAFFIC_BYTES = {
    'c5': 357.6e6 / 16,
}


def out_size(i, p, d, k, s):
    return (i + 2 * p - (d * (k - 1) + 1)) // s + 1


def flops_and_bytes(wl, n, esize):
    Ho, Wo = out_size(wl['H'], wl['p'], wl['d'], wl['k'], wl['s']), out_size(wl['W'], wl['p'], wl['d'], wl['k'], wl['s'])
    T = wl['k'] * wl['k']
    K = wl['C'] // wl['g'] * T
    fl = 2.0 * n * wl['Co'] * Ho * Wo * K
    by = n * wl['C'] * wl['H'] * wl['W'] + n * 2 * wl['dg'] * T * Ho * Wo + wl['Co'] * K + n * wl['Co'] * Ho * Wo
    if wl['mask']:
        by += n * wl['dg'] * T * Ho * Wo
    if wl['bias']:
        by += wl['Co']
    return fl, by * esize, Ho, Wo


def make_inputs(wl, n0, n1, device, dtype):
    """Samples [n0, n1) of the workload, seeded per sample so that shards are reproducible."""
    Ho, Wo = out_size(wl['H'], wl['p'], wl['d'], wl['k'], wl['s']), out_size(wl['W'], wl['p'], wl['d'], wl['k'], wl['s'])
    T = wl['k'] * wl['k']
    n = n1 - n0
    x = torch.empty(n, wl['C'], wl['H'], wl['W'], device=device, dtype=dtype)
    off = torch.empty(n, wl['dg'] * 2 * T, Ho, Wo, device=device, dtype=dtype)
    msk = torch.empty(n, wl['dg'] * T, Ho, Wo, device=device, dtype=dtype) if wl['mask'] else None
    gen = torch.Generator(device=device)
    for i in range(n):
        gen.manual_seed(n0 + i)
        x[i] = torch.randn(x.shape[1:], device=device, generator=gen)
        o = torch.randn(off.shape[1:], device=device, generator=gen) * wl['sigma']
        if wl['int_frac']:
            sel = torch.rand(o.shape, device=device, generator=gen) < wl['int_frac']
            o = torch.where(sel, o.round(), o)
        off[i] = o
        if msk is not None:
            msk[i] = torch.sigmoid(torch.randn(msk.shape[1:], device=device, generator=gen) * wl['msigma'])
    gen.manual_seed(12345)
    fan = wl['C'] // wl['g'] * T
    bound = (6.0 / fan) ** 0.5      # Kaiming-uniform
    w = ((torch.rand(wl['Co'], wl['C'] // wl['g'], wl['k'], wl['k'], device=device, generator=gen) * 2 - 1) * bound).to(dtype)
    b = (torch.rand(wl['Co'], device=device, generator=gen) * 0.2 - 0.1).to(dtype) if wl['bias'] else None
    return x, off, msk, w, b


class ClockSampler:
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile('w+', suffix='.csv', delete=False)
        try:
            self.p = subprocess.Popen(['nvidia-smi', '-i', str(index), '--query-gpu=' + self.QUERY,
                                       '--format=csv,noheader,nounits', '-lms', '20'],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [v.strip() for v in line.split(',')]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown',
                                'sw_power_cap'), c[5:9]):
                if v.lower().startswith('active'):
                    reasons.add(name)
        self.f.close()
        os.unlink(self.f.name)
        if sm:
            sm.sort()
            # median of the upper half ~ median under load (idle samples bracket the run)
            load = sm[len(sm) // 2:]
            out.update(sm_mhz=load[len(load) // 2], sm_max_mhz=max(mx), samples=len(sm))
        out['reasons'] = sorted(reasons)
        return out


def measure_msda(dev, dtype_name, peaks, reps=10):
    """Multi-scale deformable attention (the sibling sampler) at the size of a Deformable-DETR
    encoder layer on an 800x1066 image: levels 100x134, 50x67, 25x34, 13x17, every key a query,
    8 heads x 32 channels, 4 points, batch 2.  Device time of the forward kernel (median), the
    bytes it must move (value, locations, weights, output, once each) against the HBM peak, the
    corner bytes it gathers (4 per sample) per second, and a checker comparison on a slice."""
    from mmcv_b200 import _ext
    from oracle.msda import msda_forward
    dtype = torch.bfloat16 if dtype_name == 'bf16' else torch.float32
    esize = 2 if dtype_name == 'bf16' else 4
    B, M, D, P = 2, 8, 32, 4
    shapes = torch.tensor([[100, 134], [50, 67], [25, 34], [13, 17]])
    L = shapes.size(0)
    S = int(shapes.prod(1).sum())
    Q = S
    gen = torch.Generator().manual_seed(0)
    value = torch.randn(B, S, M, D, generator=gen).to(dtype)
    ref_pts = torch.rand(B, Q, 1, 1, 1, 2, generator=gen)
    loc = (ref_pts + torch.randn(B, Q, M, L, P, 2, generator=gen) * 0.03).to(dtype)
    attn = torch.rand(B, Q, M, L * P, generator=gen).softmax(-1).view(B, Q, M, L, P).to(dtype)
    starts = torch.cat((shapes.new_zeros((1,)), shapes.prod(1).cumsum(0)[:-1]))
    d = [t.to(dev) for t in (value, shapes, starts, loc, attn)]
    ts = []
    for i in range(3 + reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = _ext.ms_deform_attn_forward(*d, im2col_step=64)
        e1.record()
        torch.cuda.synchronize(dev)
        if i >= 3:
            ts.append(e0.elapsed_time(e1))
    ts.sort()
    ms = ts[len(ts) // 2]
    nq = 128   # checker slice: the first queries of the last batch entry
    ref = msda_forward(value[-1:].double(), shapes, loc[-1:, :nq].double(), attn[-1:, :nq].double())
    got = out[-1:, :nq].double().cpu()
    err = ((got - ref).norm() / ref.norm()).item()
    ok = err <= (1e-2 if dtype_name == 'bf16' else 1e-5)
    compulsory = esize * (value.numel() + loc.numel() + attn.numel() + out.numel())
    gathered = esize * B * Q * M * L * P * 4 * D
    hbm = peaks.get('hbm_gbs', 6650.0)
    return dict(workload=f'multi-scale deformable attention B={B} keys=queries={S} heads={M}x{D} levels={L} '
                         f'points={P}', dtype=dtype_name, kernel='msda_forward_kernel', ms_per_step=ms,
                compulsory_bytes=compulsory, gathered_bytes=gathered,
                roofline=dict(bound='hbm', achieved=compulsory / (ms * 1e-3) / 1e9, peak=hbm, unit='GB/s',
                              frac=compulsory / (ms * 1e-3) / 1e9 / hbm,
                              gathered_gbs=gathered / (ms * 1e-3) / 1e9,
                              note='the gather re-reads value 4*L*P/1 times per query from L2; the '
                                   'compulsory bytes alone would take '
                                   f'{compulsory / hbm / 1e6:.4f} ms'),
                parity_ok=bool(ok), parity_err=err, parity_samples=f'{nq} queries of the last batch entry')


def measure_tf32_peak(dev):
    """Dense TF32 matmul rate of this GPU (library GEMM, best of 5): the denominator of the
    3xTF32 roofline, measured the way the bf16 peak of MEASURED_PEAKS.json was."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    a = torch.randn(8192, 8192, device=dev)
    b = torch.randn(8192, 8192, device=dev)
    best = 1e9
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        a @ b
        e1.record()
        torch.cuda.synchronize(dev)
        best = min(best, e0.elapsed_time(e1))
    torch.backends.cuda.matmul.allow_tf32 = prev
    return 2 * 8192 ** 3 / (best * 1e-3) / 1e12


def cpu_reference_sample(wl, seconds_budget=20.0, max_reps=3):
    """Time the reference CPU implementation (or the C restatement) on a bounded sample of
    the workload: fp32 arithmetic on the bf16-rounded inputs, N=2 samples per call."""
    import oracle
    kind = 'reference' if oracle.have_ref() else 'port'
    torch.set_num_threads(os.cpu_count() or 1)
    n = min(2, wl['N'])
    x, off, msk, w, b = make_inputs(wl, 0, n, torch.device('cpu'), torch.bfloat16)
    f = lambda t: None if t is None else t.float()
    args = (f(x), f(off), f(msk), f(w), f(b), wl['s'], wl['p'], wl['d'], wl['g'], wl['dg'])
    fn = oracle.ref_forward if kind == 'reference' else oracle.port_forward
    fl, _, Ho, Wo = flops_and_bytes(wl, n, 2)
    best, spent, reps = None, 0.0, 0
    while reps < max_reps and spent < seconds_budget:
        t0 = time.perf_counter()
        fn(*args)
        dt = time.perf_counter() - t0
        spent += dt
        reps += 1
        best = dt if best is None else min(best, dt)
    cores = torch.get_num_threads() if kind == 'reference' else oracle.load_port().dcn_oracle_num_threads()
    return dict(value=fl / best / 1e12, unit='TFLOP/s', cores=cores, kind=kind,
                sample=f'{n} of {wl["N"]} samples, fp32 on bf16-rounded inputs, best of {reps} '
                       f'({best:.3f} s per call; gather is single-threaded in the reference, '
                       f'GEMM uses all threads)',
                seconds_per_call=best, pixels_per_s=n * Ho * Wo / best)



def abi_params(_lib, wl, n, x, off, msk, w, b, out, dtype_name, fp32_math, device_index):
    """DcnFwdParams of one layer call (the struct the public API fills)."""
    p = _lib.DcnFwdParams()
    p.input, p.offset = x.data_ptr(), off.data_ptr()
    p.mask = msk.data_ptr() if msk is not None else None
    p.weight, p.bias = w.data_ptr(), (b.data_ptr() if b is not None else None)
    p.output = out.data_ptr()
    if dtype_name == 'bf16':
        p.dtype, p.math_mode = _lib.DTYPE_BF16, _lib.MATH_AUTO
    else:
        p.dtype = _lib.DTYPE_F32
        p.math_mode = _lib.MATH_TF32X3 if fp32_math == 'tf32x3' else _lib.MATH_FFMA
    p.N, p.C, p.H, p.W, p.Co = n, wl['C'], wl['H'], wl['W'], wl['Co']
    p.kh = p.kw = wl['k']
    p.stride_h = p.stride_w = wl['s']
    p.pad_h = p.pad_w = wl['p']
    p.dil_h = p.dil_w = wl['d']
    p.groups, p.deform_groups = wl['g'], wl['dg']
    for i, s in enumerate(x.stride()):
        p.in_stride[i] = s
    p.device = device_index
    return p


def main_kernel_name(info):
    if info.path == 1:
        return 'dcn_fwd_tc2' if info.kernel_version == 2 else 'dcn_fwd_tc'
    return 'dcn_fwd_simt_tiled' if info.path == 2 else 'dcn_fwd_simt_direct'


def oracle_check(wl, x, off, msk, w, b, y, samples, dtype_name):
    """Compares samples `samples` of the device result y with the CPU checker (the compiled
    reference when present, else the C restatement) on the same inputs; bf16 results are
    checked against fp32 arithmetic on the bf16-rounded inputs.  Bounds: fp32
    max|d| <= 1e-4 max|ref| + 1e-5, bf16 relative L2 <= 2e-2."""
    import oracle
    idx = torch.tensor(sorted(set(samples)), device=x.device)
    f = lambda t: None if t is None else t.index_select(0, idx).float().cpu()
    ref = oracle.best_forward(f(x), f(off), f(msk), w.float().cpu(), None if b is None else b.float().cpu(),
                              wl['s'], wl['p'], wl['d'], wl['g'], wl['dg'])
    got = y.index_select(0, idx).float().cpu()
    if dtype_name == 'bf16':
        err = ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
        return err <= 2e-2, err
    err = (got - ref).abs().max().item()
    return err <= 1e-4 * ref.abs().max().item() + 1e-5, err


def measure_config(_lib, lib, name, dtype_name, fp32_math, dev, peaks, tf32_peak, reps=10):
    """One single-layer configuration at full size on one GPU: device time of the whole call
    and of its main kernel (median of `reps` calls after 3 warm-ups), roofline fraction of the
    layer, and a checker comparison of two samples."""
    wl = WORKLOADS[name]
    dtype = torch.bfloat16 if dtype_name == 'bf16' else torch.float32
    esize = 2 if dtype_name == 'bf16' else 4
    n = wl['N']
    x, off, msk, w, b = make_inputs(wl, 0, n, dev, dtype)
    fl, by, Ho, Wo = flops_and_bytes(wl, n, esize)
    out = torch.empty(n, wl['Co'], Ho, Wo, device=dev, dtype=dtype)
    p = abi_params(_lib, wl, n, x, off, msk, w, b, out, dtype_name, fp32_math, dev.index or 0)
    info = _lib.DcnPlanInfo()
    _lib.check(lib.dcn_fwd_plan(ctypes.byref(p), ctypes.byref(info)))
    ws = torch.empty(max(info.workspace_bytes, 256), dtype=torch.uint8, device=dev)
    sptr = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    buf = (ctypes.c_float * 3)()
    steps, mains = [], []
    for i in range(3 + reps):
        _lib.check(lib.dcn_fwd_profiled(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), ws.numel(), sptr, buf))
        if i >= 3:
            steps.append(buf[0] + buf[1] + buf[2])
            mains.append(buf[2])
    stat = ctypes.c_int32(-1)
    _lib.check(lib.dcn_read_status(ctypes.c_void_p(ws.data_ptr()), sptr, ctypes.byref(stat)))
    steps.sort(); mains.sort()
    ms, main_ms = steps[len(steps) // 2], mains[len(mains) // 2]
    hbm = peaks.get('hbm_gbs', 6650.0)
    if dtype_name == 'bf16':
        peak, peak_name = peaks.get('bf16_tflops', 1590.0), 'bf16 tensor peak (MEASURED_PEAKS.json, burst)'
    elif info.path == 1:
        peak, peak_name = tf32_peak / 3.0, f'TF32 matmul measured in this run ({tf32_peak:.0f} TFLOP/s) / 3 products'
    else:
        peak, peak_name = 148 * 128 * 2 * 1.965e9 / 1e12, 'nominal FFMA rate (148 SMs x 128 lanes x 2 x 1.965 GHz)'
    roof_ms = max(fl / (peak * 1e12), by / (hbm * 1e9)) * 1e3
    ok, err = oracle_check(wl, x, off, msk, w, b, out, [0, n - 1], dtype_name)
    return dict(workload=name + ': ' + wl['desc'], dtype=dtype_name,
                math=('bf16' if dtype_name == 'bf16' else fp32_math), kernel=main_kernel_name(info),
                ms_per_step=ms, main_kernel_ms=main_ms, tflops=fl / (ms * 1e-3) / 1e12,
                output_pixels_per_s=n * Ho * Wo / (ms * 1e-3),
                roofline=dict(bound='tensor' if fl / (peak * 1e12) >= by / (hbm * 1e9) else 'hbm',
                              layer_ms=roof_ms, frac=roof_ms / ms, frac_main_kernel=roof_ms / main_ms,
                              peak=peak, peak_name=peak_name, hbm_gbs=hbm),
                parity_ok=bool(ok and stat.value == 0), parity_err=err,
                parity_samples=[0, n - 1], launches_per_step=info.launches)


C4_LAYERS = [  # (count, C, H, W): the 13 deformable 3x3 convs of ResNet-50-DCNv2 stages 3-5
    (4, 128, 168, 100), (6, 256, 84, 50), (3, 512, 42, 25)]
C4_BATCH = 16


def c4_work(n):
    fl = by = 0.0
    for cnt, C, H, W in C4_LAYERS:
        dcn = 2.0 * n * C * H * W * C * 9
        off = 2.0 * n * 27 * H * W * C * 9
        b_dcn = 2 * (n * C * H * W * 2 + n * 27 * H * W + C * C * 9 + C)
        b_off = 2 * (n * C * H * W + 27 * C * 9 + 27 + n * 27 * H * W)
        fl += cnt * (dcn + off)
        by += cnt * (b_dcn + b_off)
    return fl, by


def run_c4(args, rank, world, local, dist_ready=False, emit=True):
    """13-layer stack through ModulatedDeformConv2dPack, bf16, N=16 (batch-sharded).  Returns the
    result line on rank 0 (and prints it when `emit`)."""
    import torch.distributed as dist
    from mmcv_b200.ops import ModulatedDeformConv2dPack
    from mmcv_b200.ops import modulated_deform_conv as mdc
    from mmcv_b200.shard import batch_shard
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1 and not dist_ready:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=dev)
    n_total = args.batch or C4_BATCH
    n0, n1 = batch_shard(n_total, rank, world)
    n = n1 - n0
    torch.manual_seed(0)
    layers, inputs = [], []
    for cnt, C, H, W in C4_LAYERS:
        for _ in range(cnt):
            m = ModulatedDeformConv2dPack(C, C, 3, padding=1, deform_groups=1, bias=True)
            m.conv_offset.weight.data.normal_(0, 0.01)
            layers.append(m.to(dev, torch.bfloat16).eval())
            gen = torch.Generator(device=dev).manual_seed(len(layers) * 1000 + n0)
            inputs.append(torch.relu(torch.randn(n, C, H, W, device=dev, generator=gen)).to(torch.bfloat16))
    stream = torch.cuda.current_stream(dev)

    def step():
        with torch.no_grad():
            for m, x in zip(layers, inputs):
                m(x)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if sampler else None
    # per stage kind, one layer timed alone (events around a single layer call)
    per_kind, idx = {}, 0
    for cnt, C, H, W in C4_LAYERS:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            layers[idx](inputs[idx])
            a.record(stream)
            for _ in range(5):
                layers[idx](inputs[idx])
            b.record(stream)
        torch.cuda.synchronize(dev)
        per_kind[f'C{C}_{H}x{W}'] = a.elapsed_time(b) / 5
        idx += cnt
    # parity, one layer of each kind, sample 0: (i) the offset branch against a plain fp32
    # convolution on the same bf16 inputs and weights; (ii) the layer's output against the CPU
    # checker fed the branch's own (bf16) offsets and mask, which isolates the deformable kernel
    parity, idx = {}, 0
    import oracle
    import torch.nn.functional as F
    for cnt, C, H, W in C4_LAYERS:
        m, x1 = layers[idx], inputs[idx][:1]
        with torch.no_grad():
            y1 = m(x1)
            br = mdc.branch_conv(mdc.shared_layout(x1), m.conv_offset, torch.bfloat16).float()
            br_ref = F.conv2d(x1.float(), m.conv_offset.weight.float(), m.conv_offset.bias.float(), padding=1)
            e_br = ((br - br_ref).norm() / br_ref.norm().clamp_min(1e-30)).item()
            br16 = br.to(torch.bfloat16).float()
            off1, msk1 = br16[:, :18].cpu(), torch.sigmoid(br16[:, 18:]).to(torch.bfloat16).float().cpu()
            ref = oracle.best_forward(x1.float().cpu(), off1, msk1, m.weight.float().cpu(),
                                      m.bias.float().cpu(), 1, 1, 1, 1, 1)
            e_y = ((y1.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-30)).item()
        parity[f'C{C}_{H}x{W}'] = dict(branch_rel_l2=e_br, layer_rel_l2=e_y, ok=bool(e_br <= 2e-2 and e_y <= 2e-2))
        idx += cnt
    # end to end: host inputs in, last layer's output out, every step
    hin = [x.cpu().pin_memory() for x in inputs]
    hout = torch.empty(inputs[-1].shape, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        with torch.no_grad():
            y = None
            for m, hx in zip(layers, hin):
                y = m(hx.to(dev, non_blocking=True))
            hout.copy_(y, non_blocking=True)

    e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for _ in range(max(1, min(args.e2e_steps, args.steps))):
        e2e_step()
    f1.record(stream)
    barrier()
    e2e_ms = f0.elapsed_time(f1) / max(1, min(args.e2e_steps, args.steps))
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank == 0:
        peaks = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json'))) if os.path.exists(
            os.path.join(ROOT, 'MEASURED_PEAKS.json')) else {}
        peak_tf, hbm = peaks.get('bf16_tflops', 1590.0), peaks.get('hbm_gbs', 6650.0)
        fl, by = c4_work(n_total)
        fl_r, _ = c4_work(n)
        roof = 0.0
        for cnt, C, H, W in C4_LAYERS:
            dcn = 2.0 * n * C * H * W * C * 9
            off = 2.0 * n * 27 * H * W * C * 9
            b_dcn = 2 * (n * C * H * W * 2 + n * 27 * H * W + C * C * 9 + C)
            b_off = 2 * (n * C * H * W + 27 * C * 9 + 27 + n * 27 * H * W)
            roof += cnt * (max(dcn / (peak_tf * 1e12), b_dcn / (hbm * 1e9)) +
                           max(off / (peak_tf * 1e12), b_off / (hbm * 1e9)))
        line = dict(
            metric='dcnv2_fwd_tflops', value=fl / (ms * 1e-3) / 1e12, unit='TFLOP/s', n_gpus=world,
            steps=args.steps, warmup=args.warmup, ms_per_step=ms, higher_is_better=True,
            scaling='strong', vs_baseline=None, dtype='bf16', data='synthetic',
            config=dict(workload='c4: 13 ModulatedDeformConv2dPack layers (ResNet-50-DCNv2 stages '
                                 '3-5), N=16, bf16, offset branch = ' + mdc.OFFSET_BRANCH + ' convolution on the shared channels-last input',
                        global_batch=n_total, parallelism=f'batch-shard x{world}, no collective',
                        l2='layer inputs 53-107 MB each, 13 distinct tensors per step (> L2)',
                        frozen_weights=bool(args.frozen_weights)),
            layer_roofline=dict(ms=roof * 1e3, frac=roof * 1e3 / ms if world == 1 else None,
                                flops=fl_r, note='sum over the 26 launches of max(FLOPs at bf16 '
                                                 'peak, compulsory bytes at HBM bandwidth)'),
            per_layer_ms=per_kind, parity=parity, parity_ok=all(v['ok'] for v in parity.values()),
            roofline=dict(bound='tensor', achieved=fl_r / (ms * 1e-3) / 1e12, peak=peak_tf,
                          unit='TFLOP/s', frac=fl_r / (ms * 1e-3) / 1e12 / peak_tf, traffic=None,
                          kernel='dcn_fwd_tc / dcn_fwd_tc2 / dcn_conv_tma (whole stack incl. the zero-bordered copies and weight tiling)'),
            e2e=dict(value=fl / (e2e_ms * 1e-3) / 1e12, unit='TFLOP/s',
                     h2d_bytes_per_step=sum(h.numel() * 2 for h in hin),
                     d2h_bytes_per_step=hout.numel() * 2, ms_per_step=e2e_ms,
                     api='mmcv_b200.ops.ModulatedDeformConv2dPack'),
            # per layer: zero-bordered copy (border + interior), branch convolution (status clear,
            # weight tiling, dcn_conv_tma), deformable kernel (status clear, weight tiling, main)
            gpu_launches=args.steps * 13 * (6 if args.frozen_weights else 8), clocks=clocks)
        if emit:
            print(json.dumps(line), flush=True)
    else:
        line = None
    if world > 1 and not dist_ready:
        dist.barrier()
        dist.destroy_process_group()
    return line


def run_backward(args, wl):
    """Forward + backward of one layer through autograd on one GPU (training step of the
    operator): device time per step and the reference CPU path on a two-sample slice."""
    import oracle
    from mmcv_b200.ops import deform_conv2d, modulated_deform_conv2d
    dev = torch.device('cuda', 0)
    dtype = torch.bfloat16 if args.dtype == 'bf16' else torch.float32
    x, off, msk, w, b = make_inputs(wl, 0, wl['N'], dev, dtype)
    leaves = [t.requires_grad_(True) for t in (x, off, msk, w, b) if t is not None]
    st, pd, dl = (wl['s'],) * 2, (wl['p'],) * 2, (wl['d'],) * 2

    def step():
        for t in leaves:
            t.grad = None
        if msk is not None:
            y = modulated_deform_conv2d(x, off, msk, w, b, st, pd, dl, wl['g'], wl['dg'])
        else:
            y = deform_conv2d(x, off, w, st, pd, dl, wl['g'], wl['dg'], False, 32)
        y.backward(torch.ones_like(y))

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    fl, _, Ho, Wo = flops_and_bytes(wl, wl['N'], 2)
    line = dict(metric='dcn_fwd_bwd_tflops', value=3 * fl / (ms * 1e-3) / 1e12, unit='TFLOP/s',
                n_gpus=1, steps=args.steps, warmup=args.warmup, ms_per_step=ms,
                higher_is_better=True, dtype=args.dtype, data='synthetic',
                config=dict(workload=args.workload + ': ' + wl['desc'] + ' ' + args.dtype +
                            ', forward + backward (3x forward FLOPs)'))
    if oracle.have_ref() and not args.no_cpu_baseline:
        ext = oracle.load_ref()
        n = min(2, wl['N'])
        c = lambda t: None if t is None else t[:n].detach().float().cpu().contiguous()
        cx, coff, cm = c(x), c(off), c(msk)
        cw, cb = w.detach().float().cpu(), (None if b is None else b.detach().float().cpu())
        gy = torch.ones(n, wl['Co'], Ho, Wo)
        e = cx.new_empty(0)
        t0 = time.perf_counter()
        oracle.ref_forward(cx, coff, cm, cw, cb, wl['s'], wl['p'], wl['d'], wl['g'], wl['dg'])
        if cm is not None:
            ext.modulated_deform_conv_backward(
                cx, cw, cb if cb is not None else e, e.clone(), coff, cm, e.clone(),
                torch.zeros_like(cx), torch.zeros_like(cw),
                torch.zeros_like(cb) if cb is not None else e.clone(), torch.zeros_like(coff),
                torch.zeros_like(cm), gy, kernel_h=wl['k'], kernel_w=wl['k'], stride_h=wl['s'],
                stride_w=wl['s'], pad_h=wl['p'], pad_w=wl['p'], dilation_h=wl['d'],
                dilation_w=wl['d'], group=wl['g'], deformable_group=wl['dg'],
                with_bias=cb is not None)
        else:
            kw = dict(kW=wl['k'], kH=wl['k'], dW=wl['s'], dH=wl['s'], padW=wl['p'], padH=wl['p'],
                      dilationW=wl['d'], dilationH=wl['d'], group=wl['g'],
                      deformable_group=wl['dg'], im2col_step=n)
            ext.deform_conv_backward_input(cx, coff, gy, torch.zeros_like(cx),
                                           torch.zeros_like(coff), cw, e.clone(), **kw)
            ext.deform_conv_backward_parameters(cx, coff, gy, torch.zeros_like(cw), e.clone(),
                                                e.clone(), scale=1.0, **kw)
        dt = time.perf_counter() - t0
        fl2, _, _, _ = flops_and_bytes(wl, n, 2)
        line['cpu_baseline'] = dict(value=3 * fl2 / dt / 1e12, unit='TFLOP/s',
                                    cores=torch.get_num_threads(), kind='reference',
                                    sample=f'{n} of {wl["N"]} samples, forward + backward, fp32, 1 call '
                                           f'({dt:.2f} s)')
    print(json.dumps(line), flush=True)


def run_reference(args, wl, rank, world):
    if rank != 0:
        return
    base = cpu_reference_sample(wl, seconds_budget=1e9, max_reps=1)   # warm the library
    times = []
    import oracle
    kind = base['kind']
    n = min(2, wl['N'])
    x, off, msk, w, b = make_inputs(wl, 0, n, torch.device('cpu'), torch.bfloat16)
    f = lambda t: None if t is None else t.float()
    a = (f(x), f(off), f(msk), f(w), f(b), wl['s'], wl['p'], wl['d'], wl['g'], wl['dg'])
    fn = oracle.ref_forward if kind == 'reference' else oracle.port_forward
    for _ in range(max(0, args.warmup - 1)):
        fn(*a)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn(*a)
    total = time.perf_counter() - t0
    fl, _, Ho, Wo = flops_and_bytes(wl, n, 2)
    val = fl * args.steps / total / 1e12
    cb = dict(base, value=val, seconds_per_call=total / args.steps)
    line = dict(impl='reference', metric='dcnv2_fwd_tflops', value=val, unit='TFLOP/s',
                n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=total / args.steps * 1e3, higher_is_better=True, scaling='strong',
                vs_baseline=None, dtype='f32', data='synthetic',
                config=dict(workload=args.workload + ': ' + wl['desc'] + ' ' + args.dtype,
                            sample=f'each step = {n} of {wl["N"]} samples on the host CPU'),
                cpu_baseline=cb,
                e2e=dict(value=val, unit='TFLOP/s', h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                output_pixels_per_s=n * Ho * Wo * args.steps / total, gpu_launches=0)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='c5', choices=sorted(WORKLOADS) + ['c4', 'msda'])
    ap.add_argument('--batch', type=int, default=0, help='override the total batch size')
    ap.add_argument('--e2e-steps', type=int, default=3)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-per-config', action='store_true',
                    help='skip the per-configuration table (c1-c4) that the default c5 run appends')
    ap.add_argument('--no-shard-check', action='store_true',
                    help='skip the checker comparison and the NCCL-gathered checksums of the shards')
    ap.add_argument('--backward', action='store_true',
                    help='time forward + backward through autograd instead of the forward')
    ap.add_argument('--frozen-weights', action='store_true',
                    help='c4 only: run the stack inside mmcv_b200.frozen_weights() (weights cast '
                         'and re-laid-out once, as in serving)')
    ap.add_argument('--counters', action='store_true',
                    help='also report the in-kernel phase counters of the first CTA (needs a library built '
                         'with DCN_B200_NVCC_FLAGS=-DDCN_B200_PHASE_COUNTERS)')
    ap.add_argument('--ablate', type=int, default=0,
                    help='timing experiments only (results are wrong): bit mask handed to '
                         'dcn_debug_configure; needs a library built with '
                         'DCN_B200_NVCC_FLAGS=-DDCN_TC2_ABLATE.  2: gather loads nothing, 8: no blend, '
                         '128: no operand store, 16: no gather body, 4: tap entries built once, '
                         '32: epilogue reads one chunk and stores nothing, 64: no MMA, 512: no weight '
                         'copies, 1024: no window copies, 256: every pass reads the window')
    ap.add_argument('--dtype', default='bf16', choices=['bf16', 'fp32'])
    ap.add_argument('--fp32-math', default='tf32x3', choices=['tf32x3', 'ffma'],
                    help='contraction arithmetic for --dtype fp32')
    args = ap.parse_args()
    if args.counters:
        os.environ['DCN_B200_COUNTERS'] = '1'
    if args.ablate:
        args.no_shard_check = args.no_per_config = args.no_cpu_baseline = True
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup
    if args.workload == 'msda':
        # the sibling sampler alone (one GPU): the two rows the default run's table carries
        if not torch.cuda.is_available():
            raise SystemExit('bench.py needs a CUDA device: there is no CPU path')
        dev = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
        torch.cuda.set_device(dev)
        peaks = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json'))) if os.path.exists(
            os.path.join(ROOT, 'MEASURED_PEAKS.json')) else {}
        if int(os.environ.get('RANK', '0')) == 0:
            rows = {dt: measure_msda(dev, dt, peaks) for dt in ('bf16', 'fp32')}
            print(json.dumps(dict(metric='msda_forward_ms', value=rows['bf16']['ms_per_step'], unit='ms',
                                  n_gpus=1, higher_is_better=False, dtype='bf16', data='synthetic',
                                  config=dict(workload=rows['bf16']['workload']), rows=rows)), flush=True)
        return
    if args.workload == 'c4':
        if args.impl == 'reference':
            raise SystemExit('the reference arm is quoted on the single-layer workloads')
        if not torch.cuda.is_available():
            raise SystemExit('bench.py needs a CUDA device: there is no CPU path')
        import contextlib
        import mmcv_b200
        with (mmcv_b200.frozen_weights() if args.frozen_weights else contextlib.nullcontext()):
            run_c4(args, int(os.environ.get('RANK', '0')), int(os.environ.get('WORLD_SIZE', '1')),
                   int(os.environ.get('LOCAL_RANK', '0')))
        return
    wl = dict(WORKLOADS[args.workload])
    if args.batch:
        wl['N'] = args.batch
    if args.backward:
        run_backward(args, wl)
        return

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))

    if args.impl == 'reference':
        run_reference(args, wl, rank, world)
        return

    import torch.distributed as dist
    from mmcv_b200 import _ext, _lib
    from mmcv_b200.ops import deform_conv2d, modulated_deform_conv2d
    lib = _lib.load()
    if args.ablate:
        _lib.check(lib.dcn_debug_configure(0, args.ablate))
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: there is no CPU path')
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=dev)

    # contiguous shard of the batch for this rank
    from mmcv_b200.shard import batch_shard
    n0, n1 = batch_shard(wl['N'], rank, world)
    per = (wl['N'] + world - 1) // world
    n = n1 - n0
    dtype = torch.bfloat16 if args.dtype == 'bf16' else torch.float32
    esize = 2 if args.dtype == 'bf16' else 4
    x, off, msk, w, b = make_inputs(wl, n0, n1, dev, dtype)
    fl_rank, by_rank, Ho, Wo = flops_and_bytes(wl, n, esize)
    fl_total, by_total, _, _ = flops_and_bytes(wl, wl['N'], esize)
    out = torch.empty(n, wl['Co'], Ho, Wo, device=dev, dtype=dtype)
    st, pd, dl = (wl['s'],) * 2, (wl['p'],) * 2, (wl['d'],) * 2

    # C-ABI parameters for the device-resident measurement (same call the public API makes)
    p = abi_params(_lib, wl, n, x, off, msk, w, b, out, args.dtype, args.fp32_math, local)
    info = _lib.DcnPlanInfo()
    _lib.check(lib.dcn_fwd_plan(ctypes.byref(p), ctypes.byref(info)))
    ws = torch.empty(max(info.workspace_bytes, 256), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)
    sptr = ctypes.c_void_p(stream.cuda_stream)

    def step():
        _lib.check(lib.dcn_fwd(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), ws.numel(), sptr))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    stat = ctypes.c_int32(-1)
    _lib.check(lib.dcn_read_status(ctypes.c_void_p(ws.data_ptr()), sptr, ctypes.byref(stat)))
    if stat.value != 0:
        raise SystemExit(f'device status {stat.value}: the kernel gave up a bounded wait')

    # per-kernel device time of the same launches (events between the kernels of a call)
    kms = [0.0, 0.0, 0.0]
    reps = max(3, min(args.steps, 10))
    buf = (ctypes.c_float * 3)()
    for _ in range(reps):
        _lib.check(lib.dcn_fwd_profiled(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), ws.numel(),
                                        sptr, buf))
        for i in range(3):
            kms[i] += buf[i] / reps
    clocks = sampler.stop() if sampler else None
    counters = None
    if args.counters and rank == 0:
        c = (ctypes.c_uint64 * 24)()
        _lib.check(lib.dcn_read_counters(ctypes.c_void_p(ws.data_ptr()), sptr, c))
        names = ['producer_other', 'table_compute', 'producer_rendezvous', 'wait_free_stage',
                 'gather_blend', 'stages', 'tables', 'publish_stage', 'mma_wait_weights',
                 'mma_wait_operand', 'mma_wait_accumulator', 'mma_issue', 'epilogue_wait',
                 'epilogue_work', 'loader_wait', 'loader_issue', 'table_load_issue',
                 'offset_prefetch']
        counters = {n: int(c[i]) for i, n in enumerate(names)}

    # End to end through the public API: every step copies the step's inputs from pinned host
    # memory to the device, runs the op, and copies the result back to pinned host memory.
    # The batch goes through in chunks on three streams (copy in, compute, copy out), so that
    # the two copy directions and the kernels overlap, as an application would arrange it.
    e2e_steps = max(1, min(args.e2e_steps, args.steps))
    hx, hoff = x.cpu().pin_memory(), off.cpu().pin_memory()
    hmsk = msk.cpu().pin_memory() if msk is not None else None
    hout = torch.empty(out.shape, dtype=dtype).pin_memory()
    h2d = (hx.numel() + hoff.numel() + (hmsk.numel() if hmsk is not None else 0)) * esize
    d2h = hout.numel() * esize
    chunk = max(1, min(n, max(1, n // 8)))
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_step():
        keep = []          # device tensors stay referenced until the step has drained
        for i0 in range(0, n, chunk):
            i1 = min(n, i0 + chunk)
            with torch.cuda.stream(s_in):
                dx = hx[i0:i1].to(dev, non_blocking=True)
                doff = hoff[i0:i1].to(dev, non_blocking=True)
                dm = hmsk[i0:i1].to(dev, non_blocking=True) if hmsk is not None else None
                ready = torch.cuda.Event()
                ready.record(s_in)
            # the chunk was allocated on s_in and is consumed on the compute stream: tell the
            # allocator, so that the blocks are not handed out again before the kernels have read them
            for t in (dx, doff, dm):
                if t is not None:
                    t.record_stream(stream)
            stream.wait_event(ready)
            if dm is not None:
                y = modulated_deform_conv2d(dx, doff, dm, w, b, st, pd, dl, wl['g'], wl['dg'])
            else:
                y = deform_conv2d(dx, doff, w, st, pd, dl, wl['g'], wl['dg'], False, 32)
            done = torch.cuda.Event()
            done.record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                hout[i0:i1].copy_(y, non_blocking=True)
                y.record_stream(s_out)
            keep.append((dx, doff, dm, y))
        stream.wait_stream(s_in)
        stream.wait_stream(s_out)
        return keep

    if args.dtype == 'fp32':
        _ext.set_fp32_math(args.fp32_math)
    keep = e2e_step()
    barrier()
    del keep
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s_in.wait_stream(stream)
    s_out.wait_stream(stream)
    f0.record(stream)
    s_in.wait_event(f0)
    for _ in range(e2e_steps):
        keep = e2e_step()
    f1.record(stream)
    barrier()
    del keep
    e2e_ms = f0.elapsed_time(f1) / e2e_steps


    # Correctness of the sharded outputs, outside the timed region: every rank compares the
    # first and the last sample of its shard with the CPU checker, and the per-sample fp64
    # checksums of all shards are gathered over NCCL; rank 0 then recomputes the other ranks'
    # shards itself (same seeds, same kernel: the checksums must agree bit for bit).
    shard_check = None
    if not args.no_shard_check:
        step()
        torch.cuda.synchronize(dev)
        ok_o, err_o = oracle_check(wl, x, off, msk, w, b, out, [0, n - 1], args.dtype)
        sums = out.double().sum(dim=(1, 2, 3))
        flag = torch.tensor([1.0 if ok_o else 0.0, err_o], device=dev, dtype=torch.float64)
        if world > 1:
            per_rank = [torch.zeros(per, device=dev, dtype=torch.float64) for _ in range(world)]
            mine = torch.zeros(per, device=dev, dtype=torch.float64)
            mine[:n] = sums
            dist.all_gather(per_rank, mine)
            flags = [torch.zeros(2, device=dev, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(flags, flag)
        else:
            per_rank, flags = [sums], [flag]
        if rank == 0:
            match = True
            for r in range(1, world):
                r0, r1 = batch_shard(wl['N'], r, world)
                xr, offr, mskr, _, _ = make_inputs(wl, r0, r1, dev, dtype)
                outr = torch.empty(r1 - r0, wl['Co'], Ho, Wo, device=dev, dtype=dtype)
                pr = abi_params(_lib, wl, r1 - r0, xr, offr, mskr, w, b, outr, args.dtype, args.fp32_math, local)
                _lib.check(lib.dcn_fwd(ctypes.byref(pr), ctypes.c_void_p(ws.data_ptr()), ws.numel(), sptr))
                torch.cuda.synchronize(dev)
                match = match and bool(torch.equal(outr.double().sum(dim=(1, 2, 3)), per_rank[r][:r1 - r0]))
                del xr, offr, mskr, outr
            allsums = torch.cat([per_rank[r][:batch_shard(wl['N'], r, world)[1] - batch_shard(wl['N'], r, world)[0]]
                                 for r in range(world)])
            shard_check = dict(
                ok=bool(match and all(f[0].item() == 1.0 for f in flags)),
                samples_checked=[[batch_shard(wl['N'], r, world)[0], batch_shard(wl['N'], r, world)[1] - 1]
                                 for r in range(world)],
                checker_err_max=max(f[1].item() for f in flags),
                checksums_gathered=int(allsums.numel()), checksums_match_single_gpu=bool(match),
                checksum_of_checksums=float(allsums.sum().item()),
                note='first and last sample of every shard against the CPU checker (bf16: relative '
                     'L2 <= 2e-2; fp32: max|d| <= 1e-4 max|ref| + 1e-5); per-sample fp64 checksums '
                     'gathered over NCCL and compared with rank 0 recomputing every other shard')

    t = torch.tensor([ms_total, e2e_ms, kms[0], kms[1], kms[2]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, k_stage, k_wt, k_main = t.tolist()
    ms_step = ms_total / args.steps

    if rank == 0:
        peaks = {}
        ppath = os.path.join(ROOT, 'MEASURED_PEAKS.json')
        if os.path.exists(ppath):
            peaks = json.load(open(ppath))
        peak_tf = peaks.get('bf16_tflops', 1590.0)
        peak_src = 'measured (MEASURED_PEAKS.json bf16_tflops, burst)' if peaks else 'fallback 1.59 PFLOP/s'
        if args.dtype == 'fp32' and info.path == 1:
            tf32 = measure_tf32_peak(dev)
            peak_tf = tf32 / 3.0
            peak_src = f'torch.matmul TF32 8192^3 measured in this run ({tf32:.0f} TFLOP/s) / 3 products'
        elif args.dtype == 'fp32':
            peak_tf = 148 * 128 * 2 * 1.965e9 / 1e12
            peak_src = 'nominal FFMA rate: 148 SMs x 128 lanes x 2 flop x 1.965 GHz'
        hbm = peaks.get('hbm_gbs', 6650.0)
        achieved = fl_rank / (k_main * 1e-3) / 1e12 if k_main > 0 else 0.0
        roof_ms = max(fl_rank / (peak_tf * 1e12), by_rank / (hbm * 1e9)) * 1e3
        # the channels-last restaging pass is a pure copy: 1 read + 1 write per input element
        stage_bytes = 2.0 * n * wl['C'] * wl['H'] * wl['W'] * (2 if args.dtype == 'bf16' else 4)
        stage_roof = (dict(bound='hbm', kernel='dcn_stage_input_cl_16bit' if args.dtype == 'bf16' else
                           'dcn_stage_input_cl_32bit', achieved=stage_bytes / (k_stage * 1e-3) / 1e9,
                           peak=hbm, unit='GB/s', frac=stage_bytes / (k_stage * 1e-3) / 1e9 / hbm)
                      if k_stage > 0 else None)
        traffic = NCU_TRAFFIC_BYTES.get(args.workload) if args.dtype == 'bf16' else None
        traffic = traffic * n if traffic is not None else None
        line = dict(
            metric='dcnv2_fwd_tflops', value=fl_total / (ms_step * 1e-3) / 1e12, unit='TFLOP/s',
            n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_step,
            higher_is_better=True, scaling='strong', vs_baseline=None,
            dtype='bf16' if args.dtype == 'bf16' else ('tf32x3' if info.path == 1 else 'f32'),
            data='synthetic',
            config=dict(workload=args.workload + ': ' + wl['desc'] + ' ' + args.dtype, global_batch=wl['N'],
                        per_gpu_batch=per, parallelism=f'batch-shard x{world}, no collective',
                        l2='inputs (GBs) larger than L2; no flush needed',
                        plan=dict(path={1: 'tcgen05', 2: 'simt_tiled', 3: 'simt_direct'}[info.path],
                                  tile=[info.tile_m, info.tile_n, info.tile_k], grid=info.grid,
                                  block=info.block, smem_bytes=info.smem_bytes,
                                  stages_input=bool(info.stages_input))),
            output_pixels_per_s=wl['N'] * Ho * Wo / (ms_step * 1e-3),
            layer_roofline=dict(ms=roof_ms, frac=roof_ms / ms_step if world == 1 else None,
                                flops=fl_rank, compulsory_bytes=by_rank,
                                note='slower of FLOPs at the bf16 peak and compulsory bytes at HBM '
                                     'bandwidth, per GPU; frac uses the whole step (all launches)'),
            kernel_ms=dict(stage_input_cl=k_stage, weight_tiles=k_wt, main=k_main),
            stage_roofline=stage_roof,
            roofline=dict(bound='tensor', achieved=achieved, peak=peak_tf, unit='TFLOP/s',
                          frac=achieved / peak_tf, traffic=traffic, peak_source=peak_src,
                          frac_of_sustained=(achieved / peaks['bf16_tflops_sustained']
                                             if 'bf16_tflops_sustained' in peaks else None),
                          kernel=main_kernel_name(info)),
            e2e=dict(value=fl_total / (e2e_ms * 1e-3) / 1e12, unit='TFLOP/s',
                     h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, ms_per_step=e2e_ms,
                     steps=e2e_steps, chunks=(n + chunk - 1) // chunk,
                     api='mmcv_b200.ops.modulated_deform_conv2d' if msk is not None
                     else 'mmcv_b200.ops.deform_conv2d'),
            gpu_launches=args.steps * info.launches,
            clocks=clocks,
        )
        if counters is not None:
            line['phase_counters_cycles_block0_last_launch'] = counters
        if not args.no_cpu_baseline:
            line['cpu_baseline'] = cpu_reference_sample(wl)
        if shard_check is not None:
            line['shard_check'] = shard_check
        if args.ablate:
            line['ablate'] = args.ablate   # a timing experiment: the outputs of this run are wrong
        if world == 1 and args.workload == 'c5' and not args.batch and not args.no_per_config:
            # every other configuration of the metric, at full size, on this GPU
            del x, off, msk, out, hx, hoff, hmsk, hout
            torch.cuda.empty_cache()
            tf32 = measure_tf32_peak(dev)
            per_config = {}
            for key, (nm, dt, fm) in {'c1_fp32_tf32x3': ('c1', 'fp32', 'tf32x3'), 'c1_fp32_ffma': ('c1', 'fp32', 'ffma'),
                                      'c2_bf16': ('c2', 'bf16', ''), 'c2_fp32_tf32x3': ('c2', 'fp32', 'tf32x3'),
                                      'c3_bf16': ('c3', 'bf16', ''), 'c3_fp32_tf32x3': ('c3', 'fp32', 'tf32x3')}.items():
                per_config[key] = measure_config(_lib, lib, nm, dt, fm, dev, peaks, tf32)
            for dt in ('bf16', 'fp32'):
                per_config['msda_' + dt] = measure_msda(dev, dt, peaks)
            c4args = argparse.Namespace(**vars(args))
            c4args.batch, c4args.steps, c4args.e2e_steps = 0, 5, 1
            c4 = run_c4(c4args, 0, 1, local, dist_ready=True, emit=False)
            per_config['c4_bf16_stack'] = dict(
                workload=c4['config']['workload'], dtype='bf16', ms_per_step=c4['ms_per_step'],
                tflops=c4['value'], per_layer_ms=c4['per_layer_ms'],
                roofline=dict(layer_ms=c4['layer_roofline']['ms'], frac=c4['layer_roofline']['frac'],
                              peak=peak_tf, peak_name='sum over the 26 launches of max(FLOPs at the bf16 '
                              'tensor peak, compulsory bytes at HBM bandwidth)'),
                parity=c4['parity'], parity_ok=c4['parity_ok'], e2e_tflops=c4['e2e']['value'])
            line['per_config'] = per_config
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == '__main__':
    main()

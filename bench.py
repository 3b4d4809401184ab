#!/usr/bin/env python
"""GPT-2 forward throughput through polygrad's instance API on the B200 backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16|fp32] [--impl b200|reference]
                    [--workload gpt2-124m|gpt2-1.5b|gemm|attention|rowops|mlp|train] [--shape MxNxK]
                    [--gather full|last|none] [--profile] [--no-cpu-baseline] [--no-sustained] [--no-configs4]

Default workload: GPT-2 124M, one step = one forward pass of 8 x 1024 token ids on every
rank (weak scaling).  Ranks hold independent replicas (weights replicated, batch rows
sharded), so the data path has no collective; with more than one rank every rank's full
fp32 logits are gathered to rank 0 inside the timed region by the library's own NCCL
send/recv on a second stream, behind the next forward (--gather last: the last position's
logits only; none: no gather).  Rank 0 prints one JSON line: `value` (with the gather) and
`value_no_gather`, both with inputs resident; `e2e` with token ids coming from page-locked
host memory and the full logits copied back to it, the copy of step i overlapping step
i+1; `roofline` for the dominant kernel (the largest projection's contraction, timed
alone); `sustained`, the same forward looped for 3 s; `cpu_baseline` (stock polygrad on one
host core, 128 tokens of sequence 0, compared with the device's logits for the same
positions); `configs4`, GPT-2 1.5B on a global batch of 64 x 1024 split over the ranks in
micro-batches of 8 (strong scaling) with the gather overlapped; `clocks` sampled through
NVML during the timed region.

The other workloads time one kernel family each: the contraction kernels on one shape or the
square sweep (gemm), the fused attention kernel (attention), the row-op kernels on a
16384 x 4096 tensor (rowops), the 784-512-10 MLP (mlp).

--impl reference times stock polygrad's CPU backend (oracle/_ref, built from polygrad's own
sources) on a bounded sample of the same workload.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ['PATH'] = os.path.join(ROOT, 'oracle', 'shim') + os.pathsep + os.environ.get('PATH', '')

WORKLOADS = {
    # BASELINE configs[3] and configs[4]; batch 8 x 1024 per plan (micro-batch of the 1.5B config)
    'gpt2-124m': dict(vocab_size=50257, n_embd=768, n_head=12, n_layer=12, max_seq_len=1024, max_batch=8),
    'gpt2-1.5b': dict(vocab_size=50257, n_embd=1600, n_head=25, n_layer=48, max_seq_len=1024, max_batch=8),
}
SEED = 1234
CPU_SAMPLE_T = 128       # tokens of one sequence that the CPU baseline of the default run computes (full width and depth)


def flops_per_token(cfg):
    d, l, v, t = cfg['n_embd'], cfg['n_layer'], cfg['vocab_size'], cfg['max_seq_len']
    per_layer = 2 * (d * 3 * d + d * d + d * 4 * d + 4 * d * d) + 4 * t * d   # projections + full T x T attention
    return l * per_layer + 2 * d * v


def read_peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.isfile(p):
        j = json.load(open(p))
        return dict(hbm_gbs=j['hbm_gbs'], bf16_tflops=j['bf16_tflops'],
                    bf16_tflops_sustained=j.get('bf16_tflops_sustained', j['bf16_tflops']), source='measured')
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source='fallback')


class ClockSampler:
    """Samples the SM clock and the clock event reasons every 10 ms during the timed
    region (NVML queries only; nothing is set)."""
    REASONS = (('hw_slowdown', 0x8), ('sw_thermal_slowdown', 0x20), ('hw_thermal_slowdown', 0x40),
               ('sw_power_cap', 0x4))

    def __init__(self, index):
        self.index, self.sm, self.bits, self.mx, self.stop_flag, self.thread, self.err = index, [], 0, None, False, None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:                       # noqa: BLE001 - any NVML failure just disables sampling
            self.err = f'NVML unavailable: {e}'
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception as e:                   # noqa: BLE001
                self.err = str(e)
                return
            time.sleep(0.01)

    def stop(self):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=2)
        if not self.sm:
            return dict(sm_mhz=None, sm_max_mhz=self.mx, reasons=[self.err or 'no samples'], samples=0)
        reasons = [n for n, bit in self.REASONS if self.bits & bit]
        return dict(sm_mhz=float(np.median(self.sm)), sm_min_mhz=float(min(self.sm)), sm_max_mhz=self.mx,
                    reasons=sorted(reasons), samples=len(self.sm))


# ── reference arm: stock polygrad on the host cores ────────────────────────
# seconds per CPU forward of one sequence of T tokens of the 124M model (measured on this pool's
# hosts; the 1.5B model costs about 12 x as much per token); used only to choose a sample size
CPU_FORWARD_S = {16: 5.0, 32: 11.0, 64: 25.0, 128: 52.0}


def workload_config(args, cfg, world):
    """The `config` object of the JSON line: the same for both arms."""
    return dict(workload=args.workload, batch_per_gpu=cfg['max_batch'], seq_len=cfg['max_seq_len'],
                parallelism=f'dp{world}',
                gemm=('bf16 operands, fp32 accumulate (tcgen05)' if args.dtype == 'bf16' else 'fp32'),
                l2='about 5 GB of intermediates written and read per step plus 1.65 GB of logits, far above the 126 MB L2',
                gather=(args.gather if world > 1 else 'none'))


def cpu_instance(cfg, t):
    from polygrad_b200 import ffi
    from polygrad_b200.instance import Instance, gpt2_init
    ref = ffi.load_reference(os.path.join(ROOT, 'oracle', '_ref', 'libpolygrad_ref.so'))
    inst = Instance.gpt2(ref, **dict(cfg, max_seq_len=t, max_batch=1))
    inst.init_params(gpt2_init(SEED))
    return inst


def cpu_forward_sample(cfg, t, tokens_row, steps, warmup):
    """Stock polygrad (CPU backend) forward on the first `t` tokens of one sequence with the
    workload's full width, depth and vocabulary.  Returns (tokens/s, seconds per forward, logits)."""
    inst = cpu_instance(cfg, t)
    inputs = inst.gpt2_inputs(np.asarray(tokens_row[:t]).reshape(1, t))
    for _ in range(max(warmup, 1)):      # the first call compiles the kernels
        inst.forward(**inputs)
    t0 = time.perf_counter()
    for _ in range(steps):
        inst.forward(**inputs)
    dt = (time.perf_counter() - t0) / steps
    logits = inst.read('output')[0].copy()
    inst.free()
    return t / dt, dt, logits


def run_reference(args, cfg, rank, world):
    if rank != 0:
        return
    from polygrad_b200 import shard
    scale = 12.0 if cfg['n_layer'] > 12 else 1.0
    budget = float(os.environ.get('POLY_B200_REF_BUDGET_S', '900'))
    t = 16
    for cand in (32, 64, 128):
        if (args.steps + args.warmup) * CPU_FORWARD_S[cand] * scale + 60 <= budget:
            t = cand
    tokens = shard.shard_tokens(SEED, 0, cfg['max_batch'], cfg['max_seq_len'], cfg['vocab_size'])
    tps, dt, _ = cpu_forward_sample(cfg, t, tokens[0], args.steps, args.warmup)
    sample = (f'each step = the first {t} tokens of 1 sequence of the workload, full {cfg["n_layer"]} layers, '
              f'd={cfg["n_embd"]}, vocab {cfg["vocab_size"]}; stock polygrad CPU backend, 1 core (it is '
              f'single-threaded by construction); the largest sample whose {args.steps}+{args.warmup} forwards fit {budget:.0f} s')
    line = dict(impl='reference', metric='gpt2_forward_tokens_per_s', value=tps, unit='tokens/s', n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=dt * 1e3, higher_is_better=True,
                scaling='weak', vs_baseline=None, dtype='f32', data='synthetic',
                config=workload_config(args, cfg, world),
                cpu_baseline=dict(value=tps, unit='tokens/s', cores=1, kind='reference', sample=sample),
                e2e=dict(value=tps, unit='tokens/s', h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


# ── product arm ─────────────────────────────────────────────────────────────
def numa_bind(local_rank):
    """Run this process (and place the page-locked buffers it allocates next) on the NUMA node
    the rank's GPU hangs off.  Reads sysfs and NVML only.  Returns a description."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(':')[0]) == 8:
            bus = bus[4:]
        node = int(open(f'/sys/bus/pci/devices/{bus}/numa_node').read())
        if node < 0:
            return 'gpu has no numa node'
        cpus = set()
        for part in open(f'/sys/devices/system/node/node{node}/cpulist').read().strip().split(','):
            lo, _, hi = part.partition('-')
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return f'node {node}: none of its cpus are available to this process'
        os.sched_setaffinity(0, cpus)
        return f'node {node}, {len(cpus)} cpus'
    except Exception as e:                           # noqa: BLE001 - binding is an optimisation only
        return f'not bound: {e}'


def comm_setup(lib, rank, world):
    """Joins the library's NCCL communicator; the id travels over a gloo group, which also
    serves the barriers and the max-over-ranks of the step times (CPU tensors only)."""
    import torch.distributed as dist
    dist.init_process_group('gloo')
    ident = (ctypes.c_ubyte * 128)()
    box = [None]
    if rank == 0:
        n = lib.poly_b200_comm_unique_id(ident, 128)
        if n <= 0:
            raise SystemExit('bench: ncclGetUniqueId failed: ' + lib.last_error())
        box[0] = bytes(ident)
    dist.broadcast_object_list(box, src=0)
    ident = (ctypes.c_ubyte * 128).from_buffer_copy(box[0])
    if lib.poly_b200_comm_init(rank, world, ident, 128) != 0:
        raise SystemExit('bench: poly_b200_comm_init failed: ' + lib.last_error())
    return dist


class Harness:
    """One rank's device, communicator and timing helpers."""

    def __init__(self, args, rank, world, local_rank):
        from polygrad_b200 import ffi, shard
        self.ffi, self.shard = ffi, shard
        self.args, self.rank, self.world, self.local_rank = args, rank, world, local_rank
        if args.dtype == 'bf16':
            os.environ['POLY_B200_GEMM'] = 'bf16'
        self.numa = numa_bind(local_rank)
        self.lib = lib = ffi.product()
        lib.poly_b200_set_device(local_rank)
        if lib.poly_cuda_init() != 0:
            raise SystemExit('bench: no usable B200: ' + lib.last_error())
        self.dist = comm_setup(lib, rank, world) if world > 1 else None

    def barrier(self):
        self.lib.poly_b200_synchronize()
        self.lib.poly_b200_comm_wait()
        if self.dist is not None:
            self.dist.barrier()

    def timed(self, fn, steps, after=None):
        """`steps` calls of fn between two events on the launching stream (`after` runs once
        before the closing event: joining other streams, waiting for copies); max over ranks."""
        lib = self.lib
        self.barrier()
        e0, e1 = lib.poly_b200_event_create(), lib.poly_b200_event_create()
        lib.poly_b200_event_record(e0)
        for _ in range(steps):
            fn()
        if after is not None:
            after()
        lib.poly_b200_event_record(e1)
        ms = lib.poly_b200_event_elapsed_ms(e0, e1)
        lib.poly_b200_event_destroy(e0); lib.poly_b200_event_destroy(e1)
        if self.dist is not None:
            ms = self.shard.max_over_ranks(self.dist, ms)
        return ms / steps

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.lib.poly_b200_comm_destroy()
            self.dist.destroy_process_group()


class Model:
    """A GPT-2 instance on the device with its inputs bound and page-locked I/O buffers."""

    def __init__(self, hx, cfg, token_rows):
        from polygrad_b200.instance import Instance, gpt2_init
        self.hx, self.lib, self.cfg = hx, hx.lib, cfg
        lib, ffi = self.lib, hx.ffi
        B, T, V = cfg['max_batch'], cfg['max_seq_len'], cfg['vocab_size']
        self.inst = Instance.gpt2(lib, **cfg)
        self.inst.init_params(gpt2_init(SEED))          # replicas: same weights on every rank
        self.inst.set_device(ffi.DEVICE_CUDA)
        self.out_idx = self.inst.bufs['output'][0]
        self.n_logits = B * T * V
        # first call: schedule + lower + compile the plan, upload inputs
        self.inst.forward(**self.inst.gpt2_inputs(token_rows[0]))
        lib.poly_b200_synchronize()
        probe = np.empty(1, np.float32)
        lib.poly_instance_readback_buf(self.inst.h, self.out_idx, probe.ctypes.data, 4)
        self.logits_ptr = lib.poly_b200_last_dtoh_src()     # where the logits live on the device
        # page-locked token ids, one buffer per micro-batch
        self.pin_tok = []
        for rows in token_rows:
            p = lib.poly_b200_host_alloc(rows.nbytes)
            ctypes.memmove(p, rows.ctypes.data, rows.nbytes)
            self.pin_tok.append(p)
        self.io = (ffi.PolyIOBinding * 1)()
        self.io[0].name = b'x'
        self.io[0].data = ctypes.cast(self.pin_tok[0], ctypes.POINTER(ctypes.c_float))
        self.tok_ptrs = (ctypes.POINTER(ctypes.c_float) * len(token_rows))(
            *[ctypes.cast(p, ctypes.POINTER(ctypes.c_float)) for p in self.pin_tok])

    def forward_resident(self):
        if self.lib.poly_instance_forward(self.inst.h, None, 0) != 0:
            raise SystemExit('bench: forward failed: ' + self.lib.last_error())

    def forward_from_host(self):
        if self.lib.poly_instance_forward(self.inst.h, self.io, 1) != 0:
            raise SystemExit('bench: forward failed: ' + self.lib.last_error())

    def readback(self, pinned):
        if self.lib.poly_instance_readback_buf(self.inst.h, self.out_idx, pinned, self.n_logits * 4) != 0:
            raise SystemExit('bench: readback failed: ' + self.lib.last_error())

    def free(self):
        for p in self.pin_tok:
            self.lib.poly_b200_host_free(p)
        self.inst.free()


def sustained_run(hx, model, cfg, seconds):
    """The same forward looped for at least `seconds`, clocks sampled throughout."""
    lib = hx.lib
    sampler = ClockSampler(hx.local_rank)
    hx.barrier()
    sampler.start()
    e0, e1 = lib.poly_b200_event_create(), lib.poly_b200_event_create()
    lib.poly_b200_event_record(e0)
    t0, steps = time.perf_counter(), 0
    while time.perf_counter() - t0 < seconds:
        for _ in range(40):
            model.forward_resident()
        steps += 40
        lib.poly_b200_synchronize()
    lib.poly_b200_event_record(e1)
    ms = lib.poly_b200_event_elapsed_ms(e0, e1)
    clocks = sampler.stop()
    lib.poly_b200_event_destroy(e0); lib.poly_b200_event_destroy(e1)
    tps = steps * cfg['max_batch'] * cfg['max_seq_len'] / (ms * 1e-3)
    peaks = read_peaks()
    tf = flops_per_token(cfg) * tps / 1e12
    return dict(seconds=ms * 1e-3, steps=steps, tokens_per_s=tps, ms_per_step=ms / steps, model_tflops=tf,
                frac_of_sustained_peak=tf / peaks['bf16_tflops_sustained'], peak_sustained=peaks['bf16_tflops_sustained'],
                peak_source=peaks['source'], clocks=clocks,
                note='one rank; every flop of the forward counted, including the row and attention kernels that '
                     'do not run on the tensor pipe')


def configs4_record(hx, steps):
    """BASELINE configs[4]: GPT-2 1.5B, bf16 policy, global batch 64 x 1024 split over the ranks
    (strong scaling) as micro-batches of 8 through one plan, every micro-batch's logits gathered
    to rank 0 behind the next micro-batch's compute."""
    lib, shard, world, rank = hx.lib, hx.shard, hx.world, hx.rank
    cfg = WORKLOADS['gpt2-1.5b']
    B, T, V = cfg['max_batch'], cfg['max_seq_len'], cfg['vocab_size']
    global_batch = 64
    n_micro = global_batch // (B * world)
    if n_micro < 1:
        return dict(skipped=f'{world} ranks x micro-batch {B} exceed the global batch {global_batch}')
    rows = [shard.shard_tokens(SEED, lib.poly_b200_shard_micro_index(rank, world, i), B, T, V) for i in range(n_micro)]
    t0 = time.perf_counter()
    model = Model(hx, cfg, rows)
    setup_s = time.perf_counter() - t0
    out_bytes = model.n_logits * 4
    root_dst = lib.poly_cuda_alloc(out_bytes * n_micro * world) if (rank == 0 and world > 1) else 0
    if rank == 0 and world > 1 and not root_dst:
        raise SystemExit('bench: cannot allocate the gather buffer: ' + lib.last_error())

    def step(gather):
        rc = lib.poly_b200_forward_microbatches(model.inst.h, b'x', model.tok_ptrs, n_micro, model.out_idx, out_bytes,
                                                root_dst or None, 0, gather)
        if rc != 0:
            raise SystemExit('bench: sharded forward failed: ' + lib.last_error())
    for _ in range(3):
        step(int(world > 1))
    lib.poly_b200_stats_reset()
    ms_plain = hx.timed(lambda: step(0), steps)
    launches = lib.stats()['launches'] // max(steps * n_micro, 1)
    ms_gather = hx.timed(lambda: step(1), steps, after=lib.poly_b200_comm_join) if world > 1 else ms_plain
    hx.barrier()
    if root_dst:
        lib.poly_cuda_free(root_dst)
    model.free()
    lib.poly_b200_trim()
    tokens = global_batch * T
    return dict(workload='gpt2-1.5b', global_batch=global_batch, seq_len=T, micro_batch=B, micro_batches_per_rank=n_micro,
                scaling='strong', steps=steps, ms_per_global_batch=ms_gather, tokens_per_s=tokens / (ms_gather * 1e-3),
                ms_no_gather=ms_plain, tokens_per_s_no_gather=tokens / (ms_plain * 1e-3),
                gather=('none (one rank holds every row)' if world == 1 else
                        f'full fp32 logits of every micro-batch to rank 0 over NCCL send/recv, overlapped with the next micro-batch'),
                gather_bytes_into_root=int(out_bytes * n_micro * (world - 1)),
                model_tflops=flops_per_token(cfg) * tokens / (ms_gather * 1e-3) / 1e12,
                launches_per_forward=int(launches), setup_s=setup_s)


def run_b200(args, cfg, rank, world, local_rank):
    hx = Harness(args, rank, world, local_rank)
    lib, shard = hx.lib, hx.shard
    B, T, V = cfg['max_batch'], cfg['max_seq_len'], cfg['vocab_size']
    tokens = shard.shard_tokens(SEED, rank, B, T, V)        # each rank's own rows of the global batch
    model = Model(hx, cfg, [tokens])
    n_logits, out_bytes = model.n_logits, model.n_logits * 4

    # the collective: every rank's full logits to rank 0 (or the last position's, --gather last)
    root_dst, last_src, gather = 0, 0, None
    if world > 1 and args.gather != 'none':
        if args.gather == 'full':
            g_bytes, g_src = out_bytes, model.logits_ptr
        else:
            # the last position of every sequence: rows of V floats, T * V apart -> one strided copy into a dense buffer
            g_bytes = B * V * 4
            last_src = lib.poly_cuda_alloc(g_bytes)
            g_src = last_src
        if rank == 0:
            root_dst = lib.poly_cuda_alloc(g_bytes * world)
            if not root_dst:
                raise SystemExit('bench: cannot allocate the gather buffer: ' + lib.last_error())

        def gather():
            if args.gather != 'full':
                if lib.poly_b200_copy_rows(last_src, model.logits_ptr + (T - 1) * V * 4, V * 4, T * V * 4, B) != 0:
                    raise SystemExit('bench: copy of the last positions failed: ' + lib.last_error())
            if lib.poly_b200_gather_async(g_src, g_bytes, root_dst or None, 0) != 0:
                raise SystemExit('bench: gather failed: ' + lib.last_error())

    def step_with_gather():
        model.forward_resident()
        gather()

    for _ in range(args.warmup):
        model.forward_resident()
        if gather is not None:
            gather()
    lib.poly_b200_stats_reset()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_compute = hx.timed(model.forward_resident, args.steps)
    st = lib.stats()
    ms_step = hx.timed(step_with_gather, args.steps, after=lib.poly_b200_comm_join) if gather is not None else ms_compute
    clocks = sampler.stop()
    launches_per_step = st['launches'] // max(args.steps, 1)

    if args.profile:
        # launch-list / ncu runs: the timed steps only
        if rank == 0:
            print(json.dumps(dict(profile=True, ms_per_step=ms_compute, launches_per_step=int(launches_per_step))), flush=True)
        hx.close()
        return

    # end to end: token ids from page-locked host memory, the full logits back into page-locked host
    # memory; the copy of step i crosses PCIe on a second stream while step i+1 computes
    pin_out = [lib.poly_b200_host_alloc(out_bytes) for _ in range(2)]
    lib.poly_b200_readback_defer(1)
    flip = [0]

    def forward_e2e():
        model.forward_from_host()
        model.readback(pin_out[flip[0]])
        flip[0] ^= 1
    for _ in range(2):
        forward_e2e()
    lib.poly_b200_readback_wait()
    e2e_steps = max(2, min(args.steps, 6))
    ms_e2e = hx.timed(forward_e2e, e2e_steps, after=lib.poly_b200_readback_wait)
    lib.poly_b200_readback_defer(0)

    tokens_per_step = B * T * world
    value = tokens_per_step / (ms_step * 1e-3)
    value_no_gather = tokens_per_step / (ms_compute * 1e-3)
    e2e_value = tokens_per_step / (ms_e2e * 1e-3)

    sustained = sustained_run(hx, model, cfg, 3.0) if not args.no_sustained else None

    # roofline of the dominant kernel: the contraction; measured live per launch
    roof = gemm_roofline(lib, args, cfg)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        t = CPU_SAMPLE_T
        tps, dt, want = cpu_forward_sample(cfg, t, tokens[0], 1, 1)
        # the same positions of the same sequence from the device run (causal: they do not depend on later tokens)
        last = pin_out[flip[0] ^ 1]
        got = np.ctypeslib.as_array(ctypes.cast(last, ctypes.POINTER(ctypes.c_float)), shape=(n_logits,))[:T * V]
        got = got.reshape(T, V)[:t]
        rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        err = np.abs(got.astype(np.float64) - want)
        cpu = dict(value=tps, unit='tokens/s', cores=1, kind='reference',
                   sample=f'the first {t} tokens of sequence 0 of the same batch, full depth/width/vocabulary, stock '
                          f'polygrad CPU backend, single-threaded by construction ({dt:.1f} s per forward)',
                   parity=dict(positions=t, max_abs_err=float(err.max()), rms_of_reference=rms,
                               max_err_over_rms=float(err.max() / rms),
                               argmax_agreement=float(np.mean(got.argmax(-1) == want.argmax(-1))),
                               bound=('2e-2 relative (bf16 policy)' if args.dtype == 'bf16' else '1e-4 relative')))

    for p in pin_out:
        lib.poly_b200_host_free(p)
    if root_dst:
        lib.poly_cuda_free(root_dst)
    if last_src:
        lib.poly_cuda_free(last_src)
    model.free()
    lib.poly_b200_trim()

    c4 = None
    if args.workload == 'gpt2-124m' and not args.no_configs4:
        c4 = configs4_record(hx, 3)

    if rank == 0:
        line = dict(metric='gpt2_forward_tokens_per_s', value=value, unit='tokens/s', n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True,
                    scaling='weak', vs_baseline=None, dtype='bf16' if args.dtype == 'bf16' else 'f32',
                    data='synthetic', config=workload_config(args, cfg, world),
                    value_no_gather=value_no_gather, ms_per_step_no_gather=ms_compute,
                    model_tflops=flops_per_token(cfg) * value_no_gather / 1e12,
                    gather=(None if gather is None else dict(
                        kind=args.gather, bytes_into_root_per_step=int(g_bytes * (world - 1)),
                        overlapped='snapshot on the main stream, NCCL send/recv on a second stream behind the next forward',
                        root_ingress_gbs=g_bytes * (world - 1) / (ms_step * 1e-3) / 1e9,
                        nvlink_peer_copy_gbs=770.0,
                        frac_of_nvlink=g_bytes * (world - 1) / (ms_step * 1e-3) / 1e9 / 770.0,
                        note='rank 0 takes in the other ranks\' logits; 770 GB/s is the peer-copy rate measured on this pool '
                             '(900 nominal per direction); from three ranks on the gather, not the forward, bounds `value`')),
                    e2e=dict(value=e2e_value, unit='tokens/s', h2d_bytes_per_step=int(tokens.nbytes),
                             d2h_bytes_per_step=int(out_bytes), ms_per_step=ms_e2e,
                             overlap='the device-to-host copy of step i runs on a second stream while step i+1 computes',
                             pcie_gbs=out_bytes / (ms_e2e * 1e-3) / 1e9, numa=hx.numa),
                    gpu_launches=int(launches_per_step * args.steps),
                    launches_per_step=int(launches_per_step),
                    clocks=clocks, roofline=roof, cpu_baseline=cpu, sustained=sustained, configs4=c4, stats=st)
        print(json.dumps(line), flush=True)
    hx.close()


def time_gemm(lib, M, N, K, bf16_policy, reps=20, bf16_buffers=False, bias=False, flags=0):
    """Device time per call of the contraction kernel(s) through the C-ABI entry
    poly_b200_gemm, operands resident, CUDA events on the launching stream.
    B is constant across calls (a weight): its bf16 copy is made once, while A is
    converted on every call, as in a model's forward."""
    from polygrad_b200.tensor import f32_to_bf16_bits
    rng = np.random.default_rng(SEED)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    if bf16_buffers:
        a, b = f32_to_bf16_bits(a), f32_to_bf16_bits(b)
    lib.poly_b200_set_gemm_policy(int(bf16_policy))
    da, db = lib.poly_cuda_alloc(a.nbytes), lib.poly_cuda_alloc(b.nbytes)
    dc = lib.poly_cuda_alloc(M * N * 4)
    dx = lib.poly_cuda_alloc(N * 4) if bias else 0
    lib.poly_cuda_copy_htod(da, a.ctypes.data, a.nbytes)
    lib.poly_cuda_copy_htod(db, b.ctypes.data, b.nbytes)
    if bias:
        lib.poly_cuda_memset(dx, 0, N * 4)

    def call():
        if flags:      # result stored as bfloat16 (1), through GELU first (3)
            rc = lib.poly_b200_gemm_ex(M, N, K, da, K, 1, db, N, 1, dc, N, dx or None, int(bf16_buffers), flags)
        else:
            rc = lib.poly_b200_gemm(M, N, K, da, K, 1, db, N, 1, dc, N, dx or None, 0, int(bf16_buffers))
        if rc != 0:
            raise SystemExit('bench: poly_b200_gemm failed: ' + lib.last_error())
    for _ in range(3):
        call()
    e0, e1 = lib.poly_b200_event_create(), lib.poly_b200_event_create()
    lib.poly_b200_event_record(e0)
    for _ in range(reps):
        call()
    lib.poly_b200_event_record(e1)
    ms = lib.poly_b200_event_elapsed_ms(e0, e1) / reps
    for d in (da, db, dc, dx):
        if d:
            lib.poly_cuda_free(d)
    return ms


def profile_traffic(name):
    """`traffic_bytes_per_launch: N` from a committed ncu summary (dram__bytes_read.sum +
    dram__bytes_write.sum of one capture of the same kernel and shape), or None."""
    import re
    path = os.path.join(ROOT, 'profiles', name)
    if not os.path.isfile(path):
        return None
    m = re.search(r'traffic_bytes_per_launch:\s*([0-9.eE+]+)', open(path).read())
    return float(m.group(1)) if m else None


def gemm_roofline(lib, args, cfg):
    """The workload's largest projection (tokens x 4d x d) alone, the way the plan runs it, against
    the tensor-pipe peak (bf16) or the fp32 FMA rate.  Under the bf16 policy that step reads
    bfloat16 activations in place, adds the bias, applies GELU and stores bfloat16 for the
    projection that follows."""
    peaks = read_peaks()
    M, K, N = cfg['max_batch'] * cfg['max_seq_len'], cfg['n_embd'], 4 * cfg['n_embd']
    bf16 = args.dtype == 'bf16'
    fused = bf16 and os.environ.get('POLY_B200_EPILOGUE', '1') != '0'
    ms = time_gemm(lib, M, N, K, bf16, bf16_buffers=bf16, bias=True, flags=3 if fused else 0)
    lib.poly_b200_set_gemm_policy(int(bf16))
    flops = 2.0 * M * N * K
    achieved = flops / (ms * 1e-3) / 1e12
    if bf16:
        peak, bound = peaks['bf16_tflops'], 'tensor'
    else:
        peak, bound = 75.0, 'fp32-cuda-core'
    prof = f'pb200_gemm_tc_{M}x{N}x{K}_bf16.md'
    traffic = profile_traffic(prof) if bf16 else None
    c_bytes = 2 if fused else 4
    return dict(bound=bound, achieved=achieved, peak=peak, unit='TFLOP/s', frac=achieved / peak, traffic=traffic,
                traffic_source=(f'profiles/{prof} (one ncu capture of this kernel and shape; not re-measured by this run)'
                                if traffic else None),
                algorithmic_bytes=(M * K * 2 + N * K * 2 + M * N * c_bytes) if bf16 else (M * K + N * K + M * N) * 4,
                algorithmic_flops=flops,
                kernel=((f'pb200_gemm_tc {M}x{N}x{K}: bf16 activations read in place, bf16 weights, bias + GELU + bf16 result'
                         if fused else
                         f'pb200_gemm_tc {M}x{N}x{K}: bf16 activations read in place, bf16 weights, fp32 result + bias')
                        if bf16 else f'fp32 contraction {M}x{N}x{K}'),
                peak_source=(peaks['source'] + ' (burst figure: the kernel is timed alone)') if bf16 else 'nominal fp32 FMA rate',
                ms_per_launch=ms)


def run_gemm_sweep(args):
    """BASELINE configs[1]: square and model-shaped contractions, fp32 and bf16."""
    from polygrad_b200 import ffi
    lib = ffi.product()
    lib.poly_b200_set_device(int(os.environ.get('LOCAL_RANK', '0')))
    if lib.poly_cuda_init() != 0:
        raise SystemExit('bench: no usable B200: ' + lib.last_error())
    peaks = read_peaks()
    if args.shape:
        shapes = [tuple(int(x) for x in args.shape.lower().split('x'))]
    else:
        shapes = [(n, n, n) for n in (1024, 2048, 4096, 8192)] + [(8192, 2304, 768), (8192, 3072, 768), (8192, 768, 3072)]
    rows = []
    for (M, N, K) in shapes:
        for mode in (['bf16', 'bf16-buffers', 'bf16-buffers-bf16out', 'bf16-buffers-gelu'] if args.dtype == 'bf16' and args.shape
                     else ['f32-simt', 'f32', 'bf16-policy', 'bf16-buffers', 'bf16-buffers-bf16out', 'bf16-buffers-gelu']):
            if mode == 'f32-simt' and M * N * K > 4096 ** 3 * 4:
                reps = 3
            else:
                reps = max(args.steps, 3)
            # 'f32': the default route (large problems: three tf32 products on the tensor cores, partial sums
            # promoted to registers); 'f32-simt': the CUDA-core kernel
            if mode == 'f32-simt':
                os.environ['POLY_B200_FP32'] = 'simt'
            flags = 3 if mode.endswith('gelu') else 1 if mode.endswith('bf16out') else 0
            if flags and (N % 4 or K < 16):
                continue
            ms = time_gemm(lib, M, N, K, mode in ('bf16-policy', 'bf16'), reps=reps, bf16_buffers=mode.startswith('bf16-buffers'),
                           bias=bool(flags), flags=flags)
            os.environ.pop('POLY_B200_FP32', None)
            tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
            # CUDA-core kernel against the nominal FMA rate; the float32 tensor-core route against what three
            # tf32 products per multiply allow (tf32 runs at half the bf16 rate: a sixth of the measured bf16 peak)
            peak = 75.0 if mode == 'f32-simt' else peaks['bf16_tflops'] / 6.0 if mode == 'f32' else peaks['bf16_tflops']
            rows.append(dict(shape=f'{M}x{N}x{K}', mode=mode, us=ms * 1e3, tflops=tf, frac_of_peak=tf / peak))
    best = max((r for r in rows if not r['mode'].startswith('f32')), key=lambda r: r['tflops'])
    print(json.dumps(dict(metric='gemm_tflops', value=best['tflops'], unit='TFLOP/s', n_gpus=1, steps=args.steps,
                          warmup=3, higher_is_better=True, dtype='bf16', data='synthetic',
                          config=dict(workload='gemm sweep', best=best['shape']),
                          roofline=dict(bound='tensor', achieved=best['tflops'], peak=peaks['bf16_tflops'], unit='TFLOP/s',
                                        frac=best['tflops'] / peaks['bf16_tflops'], traffic=None),
                          rows=rows)), flush=True)


class ResidentGraph:
    """A tensor expression realized repeatedly with every buffer resident on the device."""

    def __init__(self, lib, dev, out):
        from polygrad_b200 import ffi
        from polygrad_b200.tensor import _i64
        self.lib, self.dev = lib, dev
        n = out.numel()
        out_buf = lib.poly_buffer_by_id(dev.ctx, n, ffi.DTYPE_IDS[out.dtype])
        self.sink = lib.poly_sink1(dev.ctx, lib.poly_store_val(dev.ctx, out_buf, out.uop))
        pairs = list(out.leaves) + [(out_buf, np.empty(n, np.float32))]
        self.binds = (ffi.PolyBufferBinding * len(pairs))()
        self.n = len(pairs)
        for i, (buf, host) in enumerate(pairs):
            d = lib.poly_cuda_alloc(host.nbytes)
            if i < len(pairs) - 1:
                lib.poly_cuda_copy_htod(d, host.ctypes.data, host.nbytes)
            self.binds[i].buffer, self.binds[i].handle.ptr = buf, d
            self.binds[i].handle.nbytes, self.binds[i].handle.domain = host.nbytes, ffi.DEVICE_CUDA

    def run(self):
        if self.lib.poly_realize(self.dev.ctx, self.sink, self.binds, self.n) != 0:
            raise SystemExit('bench: poly_realize failed: ' + self.lib.last_error())

    def kernel_ms(self, reps):
        """Summed device time of the kernels of one realize (per-launch CUDA events)."""
        for _ in range(3):
            self.run()
        self.lib.poly_b200_timing_begin()
        for _ in range(reps):
            self.run()
        n = ctypes.c_int(0)
        total = self.lib.poly_b200_timing_end(ctypes.byref(n))
        return total / reps, n.value // reps

    def free(self):
        for i in range(self.n):
            self.lib.poly_cuda_free(self.binds[i].handle.ptr)


def run_rowops(args):
    """BASELINE configs[2]: row ops on a 16384 x 4096 float32 tensor ~N(0,1).  Per op: summed
    kernel time of one poly_realize, algorithmic bytes (the fused minimum: inputs once,
    outputs once) and the fraction of the measured HBM copy bandwidth."""
    from polygrad_b200 import ffi
    from polygrad_b200.tensor import Device
    lib = ffi.product()
    lib.poly_b200_set_device(int(os.environ.get('LOCAL_RANK', '0')))
    if lib.poly_cuda_init() != 0:
        raise SystemExit('bench: no usable B200: ' + lib.last_error())
    peaks = read_peaks()
    R, C = 16384, 4096
    x = np.random.default_rng(SEED).standard_normal((R, C)).astype(np.float32)
    full, red = 2.0 * x.nbytes, x.nbytes + 4.0 * R
    ops = [
        ('x*2+1', lambda t: t * 2 + 1, full), ('exp', lambda t: t.exp(), full), ('tanh', lambda t: t.tanh(), full),
        ('sum', lambda t: t.sum(-1), red), ('max', lambda t: t.max(-1), red), ('mean', lambda t: t.mean(-1), red),
        ('var', lambda t: t.var(-1), red), ('softmax', lambda t: t.softmax(-1), full),
        ('layernorm', lambda t: t.layernorm(-1, 1e-5), full),
        ('rmsnorm', lambda t: t / ((t * t).mean(-1, keepdim=True) + 1e-6).sqrt(), full),
        ('permute(1,0)', lambda t: t.permute(1, 0), full),
        ('[::-1]', lambda t: t[::-1], full), ('[:, ::-1]', lambda t: t[:, ::-1], full),
    ]
    rows = []
    for name, fn, nbytes in ops:
        dev = Device(lib, ffi.DEVICE_CUDA)
        g = ResidentGraph(lib, dev, fn(dev.tensor(x)))
        ms, launches = g.kernel_ms(max(args.steps, 3))
        g.free()
        dev.close()
        gbs = nbytes / (ms * 1e-3) / 1e9
        rows.append(dict(op=name, us=ms * 1e3, launches=launches, algorithmic_mb=nbytes / 1e6, gbs=gbs,
                         frac_of_hbm=gbs / peaks['hbm_gbs']))
    geo = float(np.exp(np.mean([np.log(r['gbs']) for r in rows])))
    print(json.dumps(dict(metric='rowops_hbm_gbs', value=geo, unit='GB/s (geometric mean over ops)', n_gpus=1,
                          steps=args.steps, warmup=3, higher_is_better=True, dtype='f32', data='synthetic',
                          config=dict(workload='row ops 16384x4096 f32', l2='536 MB per op, above the 126 MB L2'),
                          roofline=dict(bound='hbm', achieved=geo, peak=peaks['hbm_gbs'], unit='GB/s',
                                        frac=geo / peaks['hbm_gbs'], traffic=None),
                          rows=rows)), flush=True)


def run_mlp(args):
    """BASELINE configs[0]: MLP 784 -> 512 -> 10 (+ReLU), batch 256, through the instance API."""
    from polygrad_b200 import ffi
    from polygrad_b200.instance import Instance
    lib = ffi.product()
    lib.poly_b200_set_device(int(os.environ.get('LOCAL_RANK', '0')))
    if lib.poly_cuda_init() != 0:
        raise SystemExit('bench: no usable B200: ' + lib.last_error())
    x = np.random.default_rng(SEED).standard_normal((256, 784)).astype(np.float32)
    inst = Instance.mlp(lib, [784, 512, 10], 'relu', True, 256, seed=42)
    inst.set_device(ffi.DEVICE_CUDA)
    for _ in range(5):
        inst.forward(x=x)
    lib.poly_b200_synchronize()
    lib.poly_b200_stats_reset()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        if lib.poly_instance_forward(inst.h, None, 0) != 0:
            raise SystemExit('bench: forward failed')
    lib.poly_b200_synchronize()
    us = (time.perf_counter() - t0) / args.steps * 1e6
    st = lib.stats()
    cpu_us = None
    ref_path = os.path.join(ROOT, 'oracle', '_ref', 'libpolygrad_ref.so')
    if os.path.isfile(ref_path) and not args.no_cpu_baseline:
        ref = ffi.load_reference(ref_path)
        ci = Instance.mlp(ref, [784, 512, 10], 'relu', True, 256, seed=42)
        ci.forward(x=x)
        t0 = time.perf_counter()
        for _ in range(3):
            ci.forward(x=x)
        cpu_us = (time.perf_counter() - t0) / 3 * 1e6
    print(json.dumps(dict(metric='mlp_forward_us', value=us, unit='us per forward (host wall, device-resident)', n_gpus=1,
                          steps=args.steps, warmup=5, higher_is_better=False, dtype='f32', data='synthetic',
                          config=dict(workload='MLP 784-512-10 relu, batch 256'),
                          launches_per_forward=st['launches'] // max(args.steps, 1),
                          cpu_baseline=dict(value=cpu_us, unit='us per forward', cores=1, kind='reference',
                                            sample='full size') if cpu_us else None)), flush=True)


TRAIN_CFG = dict(vocab_size=2048, n_embd=256, n_head=4, n_layer=4, max_seq_len=128, max_batch=4)
# 67 M parameters (268 MB to average per step)
TRAIN_CFG_MEDIUM = dict(vocab_size=50257, n_embd=768, n_head=12, n_layer=4, max_seq_len=256, max_batch=8)


def run_train(args):
    """One optimizer step (forward, backward, SGD update in one plan) of a small GPT-2 through
    poly_instance_train_step on the device, with the CPU reference timed on the same configuration.
    On N ranks every rank steps on its own tokens and the backend averages each updated parameter over
    the ranks behind the rest of the backward pass (data-parallel SGD); the step time is the max over
    ranks and is given with and without the averaging."""
    from polygrad_b200 import ffi
    from polygrad_b200.instance import Instance, gpt2_init
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    lib = ffi.product()
    lib.poly_b200_set_device(int(os.environ.get('LOCAL_RANK', '0')))
    if lib.poly_cuda_init() != 0:
        raise SystemExit('bench: no usable B200: ' + lib.last_error())
    dist = comm_setup(lib, rank, world) if world > 1 else None
    cfg = TRAIN_CFG_MEDIUM if args.train_config == 'medium' else TRAIN_CFG
    tokens = np.random.default_rng(SEED + rank).integers(0, cfg['vocab_size'], (cfg['max_batch'], cfg['max_seq_len']))
    n_tok = cfg['max_batch'] * cfg['max_seq_len']

    def steps_of(library, device, warmup, steps, averaging=False):
        inst = Instance.gpt2(library, **cfg)
        inst.init_params(gpt2_init(SEED))
        if device != ffi.DEVICE_CPU:
            inst.set_device(device)
            library.poly_b200_set_update_averaging(1 if averaging else 0)
        inst.set_optimizer(ffi.OPTIM_SGD, 1e-6)
        io = inst.gpt2_inputs(tokens)
        losses = [inst.train_step(**io) for _ in range(warmup)]
        if device != ffi.DEVICE_CPU:
            library.poly_b200_synchronize()
            library.poly_b200_stats_reset()
            if dist is not None:
                dist.barrier()
        t0 = time.perf_counter()
        losses += [inst.train_step(**io) for _ in range(steps)]
        ms = (time.perf_counter() - t0) / steps * 1e3
        if device != ffi.DEVICE_CPU:
            library.poly_b200_set_update_averaging(0)
            if dist is not None:
                t = ctypes.c_double(ms)
                library.poly_b200_comm_max(ctypes.byref(t))
                ms = t.value
        inst.free()
        return ms, losses

    warm = max(args.warmup, 3)
    ms_alone, losses = steps_of(lib, ffi.DEVICE_CUDA, warm, args.steps)
    st = lib.stats()
    ms = ms_alone
    averaging = None
    if world > 1:
        n_par = sum(int(np.prod(shape)) for _, shape, role in _train_param_shapes(lib, cfg))
        ms, _ = steps_of(lib, ffi.DEVICE_CUDA, warm, args.steps, averaging=True)
        calls = ctypes.c_ulonglong()
        lib.poly_b200_average_trace(ctypes.byref(calls), None)
        forced = {}
        for name, flag in (('between_the_launches', '1'), ('after_the_plan', '0')):
            os.environ['POLY_B200_AVERAGE_INLINE'] = flag
            forced[name] = steps_of(lib, ffi.DEVICE_CUDA, warm, args.steps, averaging=True)[0]
        del os.environ['POLY_B200_AVERAGE_INLINE']
        averaging = dict(ms_per_step=ms, ms_per_step_without=ms_alone, ms_per_step_forced=forced,
                         allreduces_per_step=calls.value // (warm + args.steps),
                         float32_averaged_per_step=n_par + 1, mbytes_averaged_per_step=(n_par + 1) * 4 / 1e6,
                         placement='between the launches' if (n_par + 1) * 4 >= 1 << 30 else 'after the plan',
                         note='ncclAvg per parameter on a second stream; plans with 1 GB or more to average issue each '
                              'all-reduce after the parameter\'s update step, smaller ones keep their CUDA graph and '
                              'average after it')
    cpu = None
    ref_path = os.path.join(ROOT, 'oracle', '_ref', 'libpolygrad_ref.so')
    if rank == 0 and world == 1 and os.path.isfile(ref_path) and not args.no_cpu_baseline:
        cms, closses = steps_of(ffi.load_reference(ref_path), ffi.DEVICE_CPU, 1, 2)
        cpu = dict(value=n_tok / (cms * 1e-3), unit='tokens/s', cores=1, kind='reference', ms_per_step=cms,
                   sample='same configuration, 2 steps after 1 warm-up',
                   loss_rel_diff_step0=abs(losses[0] - closses[0]) / abs(closses[0]))
    if rank == 0:
        print(json.dumps(dict(metric='train_tokens_per_s', value=world * n_tok / (ms * 1e-3), unit='tokens/s', n_gpus=world,
                              steps=args.steps, warmup=warm, ms_per_step=ms, higher_is_better=True, dtype='f32',
                              data='synthetic', scaling='weak',
                              config=dict(workload='GPT-2 train step (SGD), V={vocab_size} D={n_embd} H={n_head} L={n_layer}, batch {max_batch}x{max_seq_len} per rank'.format(**cfg), **cfg),
                              timing='host wall around poly_instance_train_step (each step ends with the loss read back), max over ranks',
                              launches_per_step=st['launches'] // max(args.steps, 1),
                              precompiled_per_step=st['launches_precompiled'] // max(args.steps, 1),
                              averaging=averaging, cpu_baseline=cpu)), flush=True)
    if dist is not None:
        lib.poly_b200_synchronize()
        dist.barrier()
        lib.poly_b200_comm_destroy()
        dist.destroy_process_group()


def _train_param_shapes(lib, cfg):
    from polygrad_b200.instance import Instance
    inst = Instance.gpt2(lib, **cfg)
    out = [(n, inst.bufs[n][1], inst.bufs[n][2]) for n in inst.params]
    inst.free()
    return out


def run_attention(args):
    """The fused attention kernel alone at the GPT-2 124M layer shape (8 x 12 heads x 1024 x 64)."""
    from polygrad_b200 import ffi
    lib = ffi.product()
    lib.poly_b200_set_device(int(os.environ.get('LOCAL_RANK', '0')))
    if lib.poly_cuda_init() != 0:
        raise SystemExit('bench: no usable B200: ' + lib.last_error())
    B, H, T, hd = 8, 12, 1024, 64
    rng = np.random.default_rng(SEED)
    q, k, v = (rng.standard_normal((B, T, H, hd)).astype(np.float32) for _ in range(3))
    ar = np.arange(T, dtype=np.float32)
    mask = np.where(ar[:, None] < ar[None, :], np.float32(-1e9), np.float32(0)).astype(np.float32)
    ptrs = []
    for a in (q, k, v, mask):
        d = lib.poly_cuda_alloc(a.nbytes)
        lib.poly_cuda_copy_htod(d, a.ctypes.data, a.nbytes)
        ptrs.append(d)
    do = lib.poly_cuda_alloc(B * H * T * hd * 4)

    def call():
        if lib.poly_b200_attention(ptrs[0], ptrs[1], ptrs[2], ptrs[3], 0.125, do, B, H, T) != 0:
            raise SystemExit('bench: poly_b200_attention failed: ' + lib.last_error())
    for _ in range(3):
        call()
    e0, e1 = lib.poly_b200_event_create(), lib.poly_b200_event_create()
    lib.poly_b200_event_record(e0)
    for _ in range(args.steps):
        call()
    lib.poly_b200_event_record(e1)
    ms = lib.poly_b200_event_elapsed_ms(e0, e1) / args.steps
    flops = 4.0 * B * H * T * T * hd
    peaks = read_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    print(json.dumps(dict(metric='attention_tflops', value=tf, unit='TFLOP/s', n_gpus=1, steps=args.steps, warmup=3,
                          ms_per_step=ms, higher_is_better=True, dtype='bf16', data='synthetic',
                          config=dict(workload=f'attention {B}x{H}x{T}x{hd}, additive [T,T] mask, incl. bf16 packing of q, k, v'),
                          roofline=dict(bound='tensor', achieved=tf, peak=peaks['bf16_tflops'], unit='TFLOP/s',
                                        frac=tf / peaks['bf16_tflops'], traffic=None))), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--workload', default='gpt2-124m', choices=sorted(WORKLOADS) + ['gemm', 'attention', 'rowops', 'mlp', 'train'])
    ap.add_argument('--shape', default='', help='MxNxK for --workload gemm')
    ap.add_argument('--dtype', default='bf16', choices=['bf16', 'fp32'])
    ap.add_argument('--gather', default='full', choices=['full', 'last', 'none'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-sustained', action='store_true', help='skip the 3 s sustained loop')
    ap.add_argument('--train-config', default='small', choices=['small', 'medium'], help='size of the --workload train model')
    ap.add_argument('--no-configs4', action='store_true', help='skip the GPT-2 1.5B global-batch-64 record')
    ap.add_argument('--profile', action='store_true', help='stop after the timed steps (for ncu launch lists)')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == 'b200' else max(args.warmup, 1)
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if args.workload == 'gemm':
        return run_gemm_sweep(args)
    if args.workload == 'attention':
        return run_attention(args)
    if args.workload == 'rowops':
        return run_rowops(args)
    if args.workload == 'mlp':
        return run_mlp(args)
    if args.workload == 'train':
        return run_train(args)
    cfg = WORKLOADS[args.workload]
    if args.impl == 'reference':
        run_reference(args, cfg, rank, world)
    else:
        run_b200(args, cfg, rank, world, local_rank)


if __name__ == '__main__':
    main()

"""bench.py — headline benchmark of the B200 hot path (contract: see task statement / DESIGN.md §5).

Workload (BASELINE.json configs[2], the batched data-parallel config the metric is quoted on,
sharded 8 prompts per GPU — weak scaling; at N=8 it is exactly the 64-prompt config):
  per GPU and per step: 8 image+text prompts (one 672x672 image each, HD transform num_crops=4 ->
  5 crops, 757 image tokens) padded with random text to a 2048-token context, 256 greedy tokens.
  One step = HD transform -> CLIP ViT-L/14-336 + projector -> 32-layer prefill -> 255 decode
  steps (CUDA-graph replays) on Phi-3.5-vision, random-init bf16 weights, synthetic inputs.
`value` = batched decode tokens/s summed over all ranks, device-timed with inputs resident in HBM
(decode phase only, the reference's gen_tps definition pv:403); `e2e` = new tokens / wall time of
the PUBLIC API call a user makes — parallel.dp_generate -> api.generate_batch with prompt STRINGS and
host uint8 images (chat template, tokenizer, H2D of the images, HD transform, vision tower, prefill,
decode, D2H of the tokens, detokenisation all inside the timed region), max over ranks.
`vqa_prefill_ms` = BASELINE configs[1]: single-image VQA (336px HD crops, num_crops=4) time to
first token at batch 1.  `--impl reference` times the CPU oracle (the reference's arithmetic,
MLX itself is not installable here) on the host cores.
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
sys.path.insert(0, ROOT)

METRIC = 'batched_decode_tok_per_s'
B_PER_GPU, CTX, NEW, IMG = 8, 2048, 256, 672
KV_BYTES_PER_POS = 2 * 32 * 96 * 2          # per layer per sequence (K+V, bf16)
WEIGHT_BYTES_PER_STEP = 7_445_157_888       # SURVEY.md §8 header (decoder + lm_head, bf16)


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get('hbm_gbs', 6650.0), 'measured (MEASURED_PEAKS.json hbm_gbs)'
    return 6650.0, 'fallback (B200_PROFILING.md)'


class ClockSampler:
    def __init__(self, idx):
        self.idx, self.rows, self.proc = idx, [], None

    def start(self):
        q = 'clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,' \
            'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap'
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.idx), f'--query-gpu={q}',
                                          '--format=csv,noheader,nounits', '-lms', '200'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(',')])

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].startswith('Active') for r in self.rows)]
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': reasons, 'samples': len(sm)}


def bench_config(world):
    """the `config` object of the JSON line — identical for the b200 arm and the --impl reference arm"""
    return {'workload': 'Phi-3.5-vision batched generation: 8 image+text prompts per GPU x 2048 context x 256 '
                        'new tokens, 672x672 image, HD transform num_crops=4 (BASELINE configs[2], 64 prompts at 8 GPUs)',
            'per_gpu_batch': B_PER_GPU, 'context': CTX, 'new_tokens': NEW, 'parallelism': f'dp{world}',
            'l2_policy': 'inputs larger than L2: 7.4 GB weights + 6.8 GB KV streamed per decode step'}


def make_inputs(seed, B, ctx, n_img_tok):
    import torch
    g = torch.Generator().manual_seed(seed)
    imgs = torch.randint(0, 256, (B, IMG, IMG, 3), generator=g, dtype=torch.uint8)
    n_text = ctx - n_img_tok
    head, tail = 6, n_text - 6
    ids = torch.randint(3, 32000, (B, ctx), generator=g)
    ids[:, 0] = 1
    ids[:, head:head + n_img_tok] = -1                      # <|image_1|> placeholders (phi.py:270)
    ids[:, head + n_img_tok] = 1                            # each text chunk restarts with BOS (phi.py:265)
    assert tail > 0
    return imgs, ids


def run_cuda(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    import phi3_b200  # noqa
    from phi3_b200 import configs, weights, _lib
    from phi3_b200.model import Phi3B200
    from phi3_b200.processor import Phi3VProcessor, ByteTokenizer, hd_geometry
    from phi3_b200.api import _row_stats
    from phi3_b200 import parallel
    dev = torch.device('cuda', local)
    cfg = configs.PHI35_VISION
    w = weights.random_weights(cfg, seed=0, device=dev)     # same seed on every rank: replicated weights
    model = Phi3B200(cfg, w, device=dev)
    del w
    proc = Phi3VProcessor(ByteTokenizer(), num_crops=4, device=dev)
    ip = proc.img_processor
    geo = hd_geometry(IMG, IMG, 4)
    n_img_tok = geo['num_img_tokens']
    imgs_h, ids_h = make_inputs(1000 + rank, B_PER_GPU, CTX, n_img_tok)
    imgs_h, ids_h = imgs_h.pin_memory(), ids_h.pin_memory()
    positions = torch.nonzero(ids_h < 0)
    sizes = torch.tensor([[geo['H'], geo['W']]] * B_PER_GPU)

    def step(imgs, ids, timing=None, instrument=False):
        """one pass of the hot path over one batch; returns token history [B, NEW] on device"""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        pv = ip([imgs[i] for i in range(B_PER_GPU)])['pixel_values']
        ev[1].record()
        logits, cache = model(ids, pixel_values=pv, image_sizes=sizes, positions=positions, max_tokens=NEW,
                              logits_rows='last')
        tok = _row_stats(model, logits[:, -1, :])['argmax']
        ev[2].record()
        model.profile = [] if instrument else None
        if instrument:
            # Eager launches with an event pair around each kernel: park the GPU before EVERY step (20 ms, longer than the host needs
            # to enqueue one step's ~160 launches + 320 events) so that the host stays ahead of it and an event interval is the
            # kernel's own duration, not the host's launch gap. (One 0.15 s park at the start was enough while a step cost the host
            # less than the GPU; with the struct-argument entries the host is the slower side in eager mode and fell behind.)
            from phi3_b200.model import DecodeSession
            ses = DecodeSession(model, tok, cache, NEW - 1, False)
            for _ in range(NEW - 1):
                torch.cuda._sleep(int(0.02 * 1.9e9))
                ses.step()
            hist = ses.finish()
        else:
            hist = model.greedy_decode(tok, cache, NEW - 1, use_graph=True)
        ev[3].record()
        if timing is not None:
            timing.append(ev)
        return hist, cache

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    imgs_d, ids_d = imgs_h.to(dev), ids_h.to(dev)
    for _ in range(args.warmup):
        step(imgs_d, ids_d)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = _lib.launches
    timing = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(imgs_d, ids_d, timing)
    barrier()
    wall = time.perf_counter() - t0
    launches = _lib.launches - n0
    clocks = sampler.stop() if rank == 0 else None
    hd_ms = sum(e[0].elapsed_time(e[1]) for e in timing) / args.steps
    pre_ms = sum(e[1].elapsed_time(e[2]) for e in timing) / args.steps
    dec_ms = sum(e[2].elapsed_time(e[3]) for e in timing) / args.steps
    step_ms = sum(e[0].elapsed_time(e[3]) for e in timing) / args.steps

    # ---- e2e through the public API from host inputs: every rank calls dp_generate on the GLOBAL list of world*8 prompt
    # strings + host uint8 images (weak scaling); it shards them, runs generate_batch on its 8, and rank 0 gets the texts back.
    import torch as _t
    n_text = CTX - n_img_tok - 9                      # ByteTokenizer: 3 + n_img_tok + 6 + len(text) tokens (two chunks, two BOS)
    gtxt = _t.Generator().manual_seed(7)
    all_prompts, all_images = [], []
    for r in range(world):
        im_r, _ = make_inputs(1000 + r, B_PER_GPU, CTX, n_img_tok)
        for b in range(B_PER_GPU):
            letters = _t.randint(97, 123, (n_text,), generator=gtxt)
            all_prompts.append(bytes(letters.tolist()).decode())
            all_images.append(im_r[b].pin_memory() if r == rank else im_r[b])
    e2e_check = proc(f"<|user|>\n<|image_1|>\n{all_prompts[0]}<|end|>\n<|assistant|>\n", [all_images[0]])['input_ids'].shape[1]
    assert e2e_check == CTX, f'e2e prompt is {e2e_check} tokens, expected {CTX}'
    e2e_kw = dict(images=all_images, max_tokens=NEW, apply_chat_template=True)
    texts = parallel.dp_generate(model, proc, all_prompts, **e2e_kw)        # warm-up (slab + graph of this shape exist already)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        texts = parallel.dp_generate(model, proc, all_prompts, **e2e_kw)
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.steps
    if rank == 0:
        assert len(texts) == world * B_PER_GPU and all(isinstance(t, str) for t in texts)

    # ---- instrumented step: CUDA events around every decode-attention / skinny-GEMM launch
    roof = gemv = None
    if rank == 0:
        hist, cache = step(imgs_d, ids_d, instrument=True)
        torch.cuda.synchronize()
        peak, peak_src = peaks()
        att = [(a.elapsed_time(b), meta) for kind, a, b, meta in model.profile if kind == 'attn']
        sk = [(a.elapsed_time(b), meta) for kind, a, b, meta in model.profile if kind in ('skinny', 'mega')]
        sk_kernel = 'decode_mega_kernel (persistent layer weight stream)' if any(k == 'mega' for k, *_ in model.profile) else 'gemm_skinny_kernel (weight stream)'
        model.profile = None
        if att:
            byts = sum(m for _, m in att)
            ms = sum(t for t, _ in att)
            ach = byts / (ms * 1e-3) / 1e9
            traffic = None
            tp = os.path.join(ROOT, 'profiles', 'traffic.json')
            if os.path.exists(tp):
                traffic = json.load(open(tp)).get('attn_decode_kernel_bytes_per_launch')
            roof = {'kernel': 'attn_decode_kernel<96> (paged bf16 KV, split-KV)', 'bound': 'hbm',
                    'achieved': round(ach, 1), 'peak': peak, 'unit': 'GB/s', 'frac': round(ach / peak, 4),
                    'traffic': traffic, 'traffic_source': 'profiles/traffic.json <- ncu --set full capture of this kernel at this '
                    'shape (dram__bytes_read.sum + dram__bytes_write.sum per launch); not measured inside this run',
                    'peak_source': peak_src, 'launches': len(att),
                    'avg_us': round(1e3 * ms / len(att), 2),
                    'algorithmic_bytes_per_launch': int(byts / len(att))}
        if att:
            # the same kernel alone (no event pair per launch, no o_proj L2-prefetch duty): 32 layers' KV (6.8 GB >> L2)
            # back to back on the final cache state, so every launch streams cold pages
            from phi3_b200.model import PAGE
            B = B_PER_GPU
            past = cache.offset - 1
            qkv_t = torch.randn(B, model.qkv_dim, device=dev).to(torch.bfloat16)
            att_t = torch.empty(B, model.n_heads * model.hd, dtype=torch.bfloat16, device=dev)
            ns = model._splits(cache, B, max(1, (past + PAGE - 1) // PAGE))
            ws = torch.zeros(max(1, _lib.lib().p3_attention_decode_workspace(B, 1, model.n_heads, model.hd, ns) // 4),
                             dtype=torch.float32, device=dev)
            qp, hb = qkv_t.data_ptr(), model.n_heads * model.hd * 2
            stream = torch.cuda.current_stream().cuda_stream

            def attn_alone():
                for li in range(len(model.layers)):
                    _lib.call('p3_attention_decode', qp, qp + hb, qp + 2 * hb, model.qkv_dim, model.qkv_dim, model.qkv_dim,
                              att_t.data_ptr(), att_t.stride(0), B, 1, model.n_heads, model.n_kv, model.hd, model.scale, past,
                              cache.kv_start.data_ptr(), cache.pool[li].data_ptr(), cache.block_table.data_ptr(),
                              cache.block_table.stride(0), 1, ns, ws.data_ptr(), None, None, 0, stream)
            attn_alone()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(4):
                attn_alone()
            e1.record()
            torch.cuda.synchronize()
            us = 1e3 * e0.elapsed_time(e1) / (4 * len(model.layers))
            alone_bytes = B * past * 2 * model.n_kv * model.hd * 2
            roof['alone'] = {'avg_us': round(us, 2), 'achieved': round(alone_bytes / us / 1e3, 1),
                             'frac': round(alone_bytes / us / 1e3 / peak, 4),
                             'note': 'same kernel, 128 back-to-back launches over the 32 layers\' pages, one event pair'}
            roof['note'] = 'in-step figure: one CUDA-event pair per launch inside an eager decode pass (no PDL overlap across the events)'
        if sk:
            byts = sum(m for _, m in sk)
            ms = sum(t for t, _ in sk)
            ach = byts / (ms * 1e-3) / 1e9
            gemv = {'kernel': sk_kernel, 'bound': 'hbm', 'achieved': round(ach, 1),
                    'peak': peak, 'unit': 'GB/s', 'frac': round(ach / peak, 4), 'launches': len(sk)}

    # ---- in-graph cost of the two HBM streams of a decode step: marginal step time when one of them is skipped inside the
    # captured, PDL-chained graph (outputs are garbage, timing only). The per-launch event numbers above cannot see the overlap
    # between neighbouring kernels; these can.
    in_graph = None
    if rank == 0:
        def timed_decode(skip, steps=72, warm=8):
            model._skip = set(skip)
            try:
                pv = ip([imgs_d[i] for i in range(B_PER_GPU)])['pixel_values']
                lg, c = model(ids_d, pixel_values=pv, image_sizes=sizes, positions=positions, max_tokens=NEW, logits_rows='last')
                c.slab.session = None                                  # capture a graph with this skip set
                ses = model.decode_session(_row_stats(model, lg[:, -1, :])['argmax'], c, steps)
                for _ in range(warm):
                    ses.step()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(steps - warm):
                    ses.step()
                b.record()
                torch.cuda.synchronize()
                c.slab.session = None
                return a.elapsed_time(b) / (steps - warm)
            finally:
                model._skip = set()
        t_full, t_noattn, t_nogemm = timed_decode(()), timed_decode(('attn',)), timed_decode(('qkv', 'o', 'gu', 'down'))
        kv_bytes = B_PER_GPU * (CTX + 40) * KV_BYTES_PER_POS * 32      # mean past over the timed steps ~ CTX + 40
        gemm_bytes = 32 * 113_246_208 * 2                              # qkv + o + gate_up + down of 32 layers, bf16
        peak_, _ = peaks()
        in_graph = {'step_ms': round(t_full, 4), 'step_without_attention_ms': round(t_noattn, 4),
                    'step_without_layer_gemms_ms': round(t_nogemm, 4),
                    'attention_marginal_ms': round(t_full - t_noattn, 4), 'layer_gemm_marginal_ms': round(t_full - t_nogemm, 4),
                    'attention_frac_of_hbm_peak': round(kv_bytes / ((t_full - t_noattn) * 1e-3) / 1e9 / peak_, 4),
                    'layer_gemm_frac_of_hbm_peak': round(gemm_bytes / ((t_full - t_nogemm) * 1e-3) / 1e9 / peak_, 4),
                    'note': 'marginal cost inside the captured graph = step time minus step time with that kernel family skipped'}

    # ---- BASELINE configs[1]: single-image VQA prefill at batch 1
    vqa_ms = None
    if rank == 0:
        ids1 = ids_d[:1, :n_img_tok + 30].contiguous()
        ids1[:, n_img_tok + 6:] = torch.randint(3, 32000, (1, 24), device=dev)
        pos1 = torch.nonzero(ids1.cpu() < 0)
        ts = []
        for i in range(5):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            pv = ip([imgs_d[0]])['pixel_values']
            lg, c = model(ids1, pixel_values=pv, image_sizes=sizes[:1], positions=pos1, max_tokens=128, logits_rows='last')
            t1 = _row_stats(model, lg[:, -1, :])['argmax']
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        vqa_ms = min(ts[2:])

    # ---- BASELINE configs[4]: quantize_cache + constrained beam decoding, batch 16, beam 4 (MedQA-shaped prompts)
    cfg5 = None
    if rank == 0:
        try:
            from phi3_b200 import api as _api
            from phi3_b200.processor import Phi3FProcessor
            import numpy as _np
            rs5 = _np.random.RandomState(5)
            qs = [''.join(chr(c) for c in rs5.randint(97, 123, int(n))) for n in rs5.randint(250, 451, 16)]
            p5 = _api._apply_chat_template(qs, None, False)[0]
            class _Cfg5Tok(ByteTokenizer):
                """byte tokenizer for the prompts; the two constraint strings map to id lists of the lengths the Phi-3 tokenizer
                gives them (SURVEY par. 8d: C = 2 and C = 4 after the [1:] of pv:538), not to 4 / 22 byte tokens"""
                FIXED = {'\nThe': [29871, 13, 1576], ' The correct answer is': [29871, 450, 1959, 1234, 338]}

                def encode(self, text, add_special_tokens=True):
                    return self.FIXED.get(text) or super().encode(text, add_special_tokens)
            fproc = Phi3FProcessor(_Cfg5Tok())
            cons = [(0, '\nThe'), (100, ' The correct answer is'), 'ABCDE']
            prev_q, model.use_quantized_cache = model.use_quantized_cache, True
            model.cfg.allow_beam_with_quantized_cache = True
            ts5 = []
            for _ in range(4):                                   # best of 4: single calls vary by +-30 % (graph capture, host polling)
                torch.cuda.synchronize()
                t5 = time.perf_counter()
                out5 = _api._constrain(model, fproc, p5, cons, mute=True, verbose=False, use_beam=True, n_beam=4)
                torch.cuda.synchronize()
                ts5.append(time.perf_counter() - t5)
            model.use_quantized_cache = prev_q
            cfg5 = {'workload': 'quantize_cache=True + constrain(use_beam=True, n_beam=4), 16 prompts of 250-450 tokens, constraints '
                                "[(0,'\\nThe'),(100,' The correct answer is'),'ABCDE'] (pv:1149): 100 constrained steps, each one "
                                '[16,1+C] forward + one [64,1+C] shared-prefix beam forward', 's_per_call': round(min(ts5), 4),
                    'host_syncs_per_step': 0.125, 'rows': len(out5)}
        except Exception as e:                                  # the headline number must not depend on the extra
            cfg5 = {'error': repr(e)[:200]}

    # ---- max over ranks
    vals = torch.tensor([dec_ms, step_ms, e2e_s, pre_ms, hd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    dec_ms, step_ms, e2e_s, pre_ms, hd_ms = vals.tolist()
    tokens = world * B_PER_GPU * (NEW - 1)                  # decode-phase tokens per step (first token comes from prefill)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(steps=2)
    if rank == 0:
        line = {
            'metric': METRIC, 'value': round(tokens / (dec_ms * 1e-3), 1), 'unit': 'tok/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(dec_ms, 3), 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16',
            'data': 'synthetic (random-init bf16 weights, random uint8 images and token ids; no network)',
            'config': bench_config(world),
            'whole_step_ms': round(step_ms, 2), 'hd_transform_ms': round(hd_ms, 3),
            'vision_prefill_ms': round(pre_ms, 2), 'decode_ms_per_token': round(dec_ms / (NEW - 1), 4),
            'vqa_prefill_ms': None if vqa_ms is None else round(vqa_ms, 3), 'constrain_cfg5': cfg5,
            'e2e': {'value': round(world * B_PER_GPU * NEW / e2e_s, 1), 'unit': 'tok/s',
                    'h2d_bytes_per_step': int(imgs_h.numel() + ids_h.numel() * 8 * 3),
                    'd2h_bytes_per_step': int(B_PER_GPU * NEW * 4), 's_per_step': round(e2e_s, 4),
                    'call': 'parallel.dp_generate -> api.generate_batch(prompt strings, host uint8 images): new tokens / wall '
                            'time of the whole call incl. tokenizer, H2D, HD transform, vision tower, prefill, decode, D2H, detokenise'},
            'gpu_launches': int(launches), 'clocks': clocks, 'roofline': roof, 'roofline_skinny_gemm': gemv,
            'decode_step_in_graph': in_graph,
            'cpu_baseline': cpu, 'wall_s_timed_region': round(wall, 3),
        }
        _emit(line)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(steps=2, threads=None):
    """The CPU oracle (op-for-op restatement of the reference, fp32) on the host cores: B=8 decode
    steps against a 2048-token synthetic KV cache (bounded sample of the same workload)."""
    import torch
    from phi3_b200 import configs
    from oracle.phi3_oracle import Phi3Oracle, KVCache, Mask4D, SuRoPE
    threads = threads or os.cpu_count()
    torch.set_num_threads(threads)
    cfg = configs.PHI35_MINI
    t0 = time.perf_counter()
    from phi3_b200.weights import _names
    w = {}
    g = torch.Generator().manual_seed(0)
    for name, shape, kind in _names(cfg, None, False):
        t = torch.empty(shape, dtype=torch.float32)
        t.normal_(0, 0.02, generator=g) if kind in ('lin', 'res') else t.normal_(1.0 if kind == 'norm' else 0.0, 0.1 if kind == 'norm' else 1.0, generator=g)
        w[name] = t
    o = Phi3Oracle(cfg, w, prec='fp32')
    B, S = B_PER_GPU, CTX
    cache = [KVCache(cfg, B, S, NEW, 'fp32') for _ in range(cfg.num_hidden_layers)]
    for c in cache:
        c.k = torch.randn(c.shape) * 0.5
        c.v = torch.randn(c.shape) * 0.5
        c.offset, c.prompt_done = S, True
    o._masker = Mask4D(S + NEW, None)
    o._roper = SuRoPE(cfg, S + NEW, None)
    setup = time.perf_counter() - t0
    tok = torch.randint(3, 32000, (B, 1))
    ts = []
    for i in range(steps + 1):
        t1 = time.perf_counter()
        lg, cache = o(tok, cache=cache)
        tok = lg[:, -1].argmax(-1)[:, None]
        ts.append(time.perf_counter() - t1)
    s = min(ts[1:])
    return {'value': round(B / s, 3), 'unit': 'tok/s', 'cores': threads, 'kind': 'port',
            'sample': f'decode phase of the bench workload on one GPU share: batch {B}, {steps} greedy decode steps at a {S}-token '
                      f'synthetic fp32 KV cache through the 32-layer Phi-3.5 LM backbone (the same architecture in the mini and vision '
                      f'checkpoints), reference semantics: dense mask, fp32 KV, lm_head on every position; setup {setup:.0f}s excluded',
            's_per_step': round(s, 3)}


def run_reference(args):
    rank = int(os.environ.get('RANK', 0))
    if rank != 0:
        return
    cb = cpu_baseline(steps=max(1, args.steps))
    line = {'impl': 'reference', 'metric': METRIC, 'value': cb['value'], 'unit': 'tok/s', 'n_gpus': int(os.environ.get('WORLD_SIZE', 1)),
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(1e3 * cb['s_per_step'], 1),
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'config': bench_config(int(os.environ.get('WORLD_SIZE', 1))),
            'reference_impl': 'CPU oracle (op-for-op restatement of the reference; MLX itself is not installable offline) on a '
                              'bounded sample of the workload, see cpu_baseline.sample',
            'cpu_baseline': cb, 'e2e': {'value': cb['value'], 'unit': 'tok/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}
    _emit(line)


_RESULT_FD = None


def _claim_stdout():
    """stdout must carry exactly one line, the JSON result: keep a private copy of fd 1 for it and point fd 1 at stderr, so
    library chatter (e.g. NCCL's version banner, which ignores NCCL_DEBUG_FILE) cannot interleave with the result."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def _emit(line):
    data = (json.dumps(line) + '\n').encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


# ------------------------------------------------------------------------------------------------ --arch tagenex
def _engine_model_numbers(m, B, L, CTX_D, NEW_D, vocab, args, hbm, tf):
    """prefill and decode throughput of one engine model (B requests of L prompt tokens; decode at CTX_D tokens of context) and
    the time of every kernel family with its achieved FLOP/s (prefill) or bytes/s (decode) against the measured peaks.
    Device-timed with CUDA events after warm-up. -> (prompts, numbers)"""
    import torch
    from phi3_b200.engine import Engine

    def timed(fn, n):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, vocab, (L,), generator=g).tolist() for _ in range(B)]
    eng = Engine(m, B * (CTX_D + 64), B)

    def prefill():
        eng.step([(i, prompts[i], [L - 1]) for i in range(B)], list(range(B)))
    ms_pf = timed(prefill, args.steps)
    m.profile = []
    prefill()
    torch.cuda.synchronize()
    fam = {}
    for kind, a, b, fl, by in m.profile:
        f = fam.setdefault(kind, [0.0, 0, 0, 0])
        f[0] += a.elapsed_time(b); f[1] += fl; f[2] += by; f[3] += 1
    m.profile = None
    kern_pf = {k: dict(ms=round(v[0], 3), launches=v[3], tflops=round(v[1] / v[0] / 1e9, 1),
                       frac_of_measured_bf16=round(v[1] / v[0] / 1e9 / tf, 3),
                       **({'gbs': round(v[2] / v[0] / 1e6, 1), 'frac_of_measured_hbm': round(v[2] / v[0] / 1e6 / hbm, 3)}
                          if v[2] and not v[1] else {})) for k, v in fam.items()}
    # decode: B sequences at CTX_D tokens of context, one token each per step
    eng.step([(i, prompts[i][:CTX_D - NEW_D - 8], []) for i in range(B)])
    tok = [1] * B

    def decode():
        eng.step([(i, [tok[i]], [0]) for i in range(B)])
    for _ in range(3):
        decode()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(NEW_D):
        decode()
    e1.record()
    torch.cuda.synchronize()
    ms_dec = e0.elapsed_time(e1) / NEW_D
    m.profile = []
    decode()
    torch.cuda.synchronize()
    fam = {}
    for kind, a, b, fl, by in m.profile:
        f = fam.setdefault(kind, [0.0, 0, 0, 0])
        f[0] += a.elapsed_time(b); f[1] += fl; f[2] += by; f[3] += 1
    m.profile = None
    kern_dec = {k: dict(ms=round(v[0], 3), launches=v[3], gbs=round(v[2] / v[0] / 1e6, 1),
                        frac_of_measured_hbm=round(v[2] / v[0] / 1e6 / hbm, 3)) for k, v in fam.items()}
    return prompts, dict(prefill_tok_s=round(B * L / ms_pf * 1e3), prefill_ms=round(ms_pf, 2), decode_tok_s=round(B / ms_dec * 1e3),
                         decode_ms_per_step=round(ms_dec, 3), prefill_kernels=kern_pf, decode_kernels=kern_dec)


def _tagenex_cfg(width, heads, kv, dim, ff, layers, window, vocab, moe):
    att = {'type': 'attention', 'mixer': {'heads': heads, 'kv_heads': kv, 'dim': dim, 'vdim': dim, 'scale': dim ** -0.5,
                                          'v_mix': True, 'mask': {'size': window}}}
    dense = {'kind': 'dense', 'ff': ff, 'limit': 7.0}
    mix = {'kind': 'moe', 'expert': {'ff': ff // 4, 'limit': 7.0}, 'router': {'experts': 8, 'top': 2}}
    return {'architecture': 'Tagenex', 'vocab': vocab, 'width': width, 'norm': {'eps': 1e-5},
            'layers': [dict(att, mlp=(mix if (moe and i % 2) else dense)) for i in range(layers)]}


def run_tagenex(args):
    """Throughput of the Tagenex design on the continuous-batching engine at layer sizes of a real model (random weights, bf16
    serving mode), beside Phi-3 (the closest existing model: same width, heads, feed-forward size and depth) on its own path.
    One JSON line: per size prefill tok/s and decode tok/s of both, and for Tagenex the time of every kernel family with its
    achieved FLOP/s or bytes/s against the measured peaks. Device-timed with CUDA events after warm-up; the weights plus the
    activations of a step exceed L2 at the large sizes."""
    import torch
    import phi3_b200  # noqa: F401
    from phi3_b200 import configs, weights
    from phi3_b200.engine import Engine
    from phi3_b200.tagenex import TagenexB200
    from phi3_b200.model import Phi3B200
    hbm, _ = peaks()
    tf = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json'))).get('bf16_tflops', 1590.0) if os.path.exists(
        os.path.join(ROOT, 'MEASURED_PEAKS.json')) else 1590.0
    dev = torch.device('cuda:0')
    sizes = [dict(name='w3072_h32x96_ff8192_L4', width=3072, heads=32, kv=32, dim=96, ff=8192, layers=4, window=1024, moe=False),
             dict(name='w3072_h32x96_ff8192_L4_b16', width=3072, heads=32, kv=32, dim=96, ff=8192, layers=4, window=1024, moe=False,
                  batch=16),
             dict(name='w3072_h32x96_kv8_moe_L4', width=3072, heads=32, kv=8, dim=96, ff=8192, layers=4, window=1024, moe=True),
             dict(name='w1024_h8x128_kv2_moe_L4', width=1024, heads=8, kv=2, dim=128, ff=4096, layers=4, window=512, moe=True)]
    vocab, L, CTX_D, NEW_D = 32064, 2048, 2048, 32

    def timed(fn, n):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    out = []
    for sz in sizes:
        B = sz.get('batch', 4)
        cfg = _tagenex_cfg(sz['width'], sz['heads'], sz['kv'], sz['dim'], sz['ff'], sz['layers'], sz['window'], vocab, sz['moe'])
        m = TagenexB200(cfg, weights.random_tagenex_weights(cfg, 0, device=dev), dtype=torch.bfloat16)
        prompts, nums = _engine_model_numbers(m, B, L, CTX_D, NEW_D, vocab, args, hbm, tf)
        row = dict(size=sz['name'], batch=B, prompt=L, tagenex=nums)
        del m
        torch.cuda.empty_cache()
        if sz['kv'] == sz['heads'] and sz['dim'] == 96 and not sz['moe']:
            # Phi-3 at equal size: same width, heads, head size, feed-forward and depth (full attention instead of a window)
            pc = configs.with_overrides(configs.PHI35_MINI, hidden_size=sz['width'], num_attention_heads=sz['heads'],
                                        num_key_value_heads=sz['kv'], intermediate_size=sz['ff'], num_hidden_layers=sz['layers'],
                                        vocab_size=vocab)
            pm = Phi3B200(pc, weights.random_weights(pc, seed=0, device=dev))
            ids = torch.tensor(prompts)

            def p_prefill():
                lg, c = pm(ids, max_tokens=NEW_D + 8, logits_rows='last')
                c.release()
            ms_ppf = timed(p_prefill, args.steps)
            lg, cache = pm(ids[:, :CTX_D - NEW_D - 8], max_tokens=NEW_D + 16, logits_rows='last')
            ses = pm.decode_session(lg[:, -1].argmax(-1), cache, NEW_D + 8)
            for _ in range(3):
                ses.step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(NEW_D):
                ses.step()
            e1.record()
            torch.cuda.synchronize()
            row['phi3_equal_size'] = dict(prefill_tok_s=round(B * L / ms_ppf * 1e3), prefill_ms=round(ms_ppf, 2),
                                          decode_tok_s=round(B / (e0.elapsed_time(e1) / NEW_D) * 1e3),
                                          decode_ms_per_step=round(e0.elapsed_time(e1) / NEW_D, 3), note='CUDA-graph decode loop')
            ses.finish()
            cache.release()
            del pm
            torch.cuda.empty_cache()
        out.append(row)
    _emit({"metric": "tagenex_prefill_decode_tok_per_s", 'arch': 'tagenex', 'dtype': 'bf16', 'data': 'synthetic', 'n_gpus': 1,
          'steps': args.steps, 'warmup': max(3, args.warmup), 'peaks': {'hbm_gbs': hbm, 'bf16_tflops': tf}, 'sizes': out})


# ------------------------------------------------------------------------------------------------ --arch tapalix
def _tapalix_cfg(width, heads, dim, rot, vdim, rank, eff, experts, top, shared, layers, vocab):
    rotc = {'base': 10000.0, 'dims': rot, 'scaling': {'factor': 4.0, 'original': 4096, 'fast': 32.0, 'slow': 1.0}}
    la = {'type': 'latent_attention', 'mixer': {'heads': heads, 'dim': dim, 'rot_dim': rot, 'vdim': vdim, 'kv_rank': rank,
                                                'scale': (dim + rot) ** -0.5, 'rot': rotc}}
    la2 = {'type': 'latent_attention_2', 'mixer': {'heads': heads, 'dim': dim + rot, 'vdim': vdim, 'kv_rank': rank + rot,
                                                   'scale': (dim + rot) ** -0.5}}
    moe = {'kind': 'moe', 'expert': {'ff': eff}, 'router': {'experts': experts, 'top': top, 'scale': 2.0,
                                                              'groups': {'count': 4, 'keep': 2}}, 'shared': {'ff': shared}}
    return {'architecture': 'Tapalix', 'vocab': vocab, 'width': width, 'norm': {'eps': 1e-5}, 'embedding': {'scale': width ** 0.5},
            'layers': [dict(la if i % 2 else la2, mlp=moe) for i in range(layers)],
            'loop': {'start': 1, 'stop': layers - 1, 'times': 2}, 'logit_scale': 1.0, 'logit_softcap': 30.0}


def run_tapalix(args):
    """Throughput of the Tapalix design on the continuous-batching engine at layer sizes of a real model (random weights, bf16
    serving mode), beside Tagenex, the closest existing model (same engine, page pool, product kernels and expert path), at equal
    width, head count, per-head key size, expert sizes and number of layer runs. One JSON line: per size the prefill and decode
    tok/s of both and, per kernel family, time and achieved FLOP/s (prefill) or bytes/s (decode) against the measured peaks."""
    import torch
    import phi3_b200  # noqa: F401
    from phi3_b200 import weights
    from phi3_b200.tagenex import TagenexB200
    from phi3_b200.tapalix import TapalixB200
    hbm, _ = peaks()
    tf = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json'))).get('bf16_tflops', 1590.0) if os.path.exists(
        os.path.join(ROOT, 'MEASURED_PEAKS.json')) else 1590.0
    dev = torch.device('cuda:0')
    # latent rows of 128 numbers run on the tensor-core attention kernels, rows of 256 on the fp32 ones
    sizes = [dict(name='w2048_h16x(64+32)_r96_e8x1408_L4', width=2048, heads=16, dim=64, rot=32, vdim=64, rank=96, eff=1408, experts=8,
                  top=2, shared=2816, layers=4),
             dict(name='w2048_h16x(64+32)_r96_e8x1408_L4_b16', width=2048, heads=16, dim=64, rot=32, vdim=64, rank=96, eff=1408,
                  experts=8, top=2, shared=2816, layers=4, batch=16),
             dict(name='w3072_h32x(64+32)_r96_e16x1024_L4', width=3072, heads=32, dim=64, rot=32, vdim=96, rank=96, eff=1024, experts=16,
                  top=4, shared=2048, layers=4),
             dict(name='w2048_h16x(128+64)_r192_e8x1408_L4', width=2048, heads=16, dim=128, rot=64, vdim=128, rank=192, eff=1408,
                  experts=8, top=2, shared=2816, layers=4)]
    vocab, L, CTX_D, NEW_D = 32064, 2048, 2048, 32
    out = []
    for sz in sizes:
        B = sz.get('batch', 4)
        cfg = _tapalix_cfg(sz['width'], sz['heads'], sz['dim'], sz['rot'], sz['vdim'], sz['rank'], sz['eff'], sz['experts'], sz['top'],
                           sz['shared'], sz['layers'], vocab)
        m = TapalixB200(cfg, weights.random_tapalix_weights(cfg, 0, device=dev), dtype=torch.bfloat16)
        _, nums = _engine_model_numbers(m, B, L, CTX_D, NEW_D, vocab, args, hbm, tf)
        runs = len(m.cfg.runs)
        row = dict(size=sz['name'], batch=B, prompt=L, layer_runs=runs, tapalix=nums)
        del m
        torch.cuda.empty_cache()
        # Tagenex at equal size: as many layers as Tapalix has layer runs, every layer a mixture of the same experts, grouped-query
        # attention with as many heads of the same key size, no window shorter than the context
        d = sz['dim'] + sz['rot']
        if d <= 128:
            att = {'type': 'attention', 'mixer': {'heads': sz['heads'], 'kv_heads': max(1, sz['heads'] // 8), 'dim': d, 'vdim': sz['vdim'],
                                                  'scale': d ** -0.5, 'v_mix': False}}
            mix = {'kind': 'moe', 'expert': {'ff': sz['eff'], 'limit': 7.0}, 'router': {'experts': sz['experts'], 'top': sz['top']}}
            tcfg = {'architecture': 'Tagenex', 'vocab': vocab, 'width': sz['width'], 'norm': {'eps': 1e-5},
                    'layers': [dict(att, mlp=mix) for _ in range(runs)]}
            tm = TagenexB200(tcfg, weights.random_tagenex_weights(tcfg, 0, device=dev), dtype=torch.bfloat16)
            _, row['tagenex_equal_size'] = _engine_model_numbers(tm, B, L, CTX_D, NEW_D, vocab, args, hbm, tf)
            del tm
            torch.cuda.empty_cache()
        out.append(row)
    _emit({"metric": "tapalix_prefill_decode_tok_per_s", 'arch': 'tapalix', 'dtype': 'bf16', 'data': 'synthetic', 'n_gpus': 1,
          'steps': args.steps, 'warmup': max(3, args.warmup), 'peaks': {'hbm_gbs': hbm, 'bf16_tflops': tf}, 'sizes': out})


# ------------------------------------------------------------------------------------------------ --arch dugalix
def _dugalix_cfg(width, heads, kv, dim, window, keep, mh, mdim, mvdim, ff, eff, experts, identity, top, shared, layers, vocab):
    rot = lambda dims, factor=None: {'base': 500000.0, 'dims': dims, **({'scaling': {'factor': factor}} if factor else {})}
    par = {'type': 'parallel',
           'mixer': {'left': {'heads': heads, 'kv_heads': kv, 'dim': dim, 'vdim': dim, 'scale': dim ** -0.5,
                              'mask': {'size': window, 'keep_first': keep}, 'rot': rot(dim, 4.0)},
                     'right': {'heads': mh, 'dim': mdim, 'vdim': mvdim, 'gate_cap': 15.0}, 'left_scale': 0.7, 'right_scale': 0.7}}
    sig = {'type': 'attention', 'mixer': {'heads': heads, 'kv_heads': kv, 'dim': dim, 'vdim': dim, 'scale': dim ** -0.5,
                                          'mask': {'size': window}, 'rot': rot(dim // 2)}}
    dense = {'kind': 'dense', 'ff': ff}
    moe = {'kind': 'moe', 'expert': {'ff': eff}, 'router': {'experts': experts, 'identity': identity, 'top': top,
                                                              'groups': {'count': 4, 'keep': 2}}, 'shared': {'ff': shared}}
    return {'architecture': 'Dugalix', 'vocab': vocab, 'width': width, 'norm': {'eps': 1e-5}, 'residual_mult': 0.6,
            'layers': [dict(sig if i % 2 else par, mlp=(moe if i else dense)) for i in range(layers)]}


def run_dugalix(args):
    """Throughput of the Dugalix design on the continuous-batching engine at layer sizes of a real model (random weights, bf16
    serving mode), beside Tagenex, the closest existing model (same engine, page pool, product kernels, windowed attention and
    expert path), at equal width, depth, attention shape, window and expert sizes. One JSON line: per size the prefill and decode
    tok/s of both and, per kernel family, time and achieved FLOP/s (prefill) or bytes/s (decode) against the measured peaks."""
    import torch
    import phi3_b200  # noqa: F401
    from phi3_b200 import weights
    from phi3_b200.tagenex import TagenexB200
    from phi3_b200.dugalix import DugalixB200
    hbm, _ = peaks()
    tf = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json'))).get('bf16_tflops', 1590.0) if os.path.exists(
        os.path.join(ROOT, 'MEASURED_PEAKS.json')) else 1590.0
    dev = torch.device('cuda:0')
    sizes = [dict(name='w2048_h16x128_kv4_m8x128x256_e8x1408_L4', width=2048, heads=16, kv=4, dim=128, window=1024, keep=64, mh=8,
                  mdim=128, mvdim=256, ff=8192, eff=1408, experts=8, identity=8, top=2, shared=2816, layers=4),
             dict(name='w2048_h16x128_kv4_m8x128x256_e8x1408_L4_b16', width=2048, heads=16, kv=4, dim=128, window=1024, keep=64, mh=8,
                  mdim=128, mvdim=256, ff=8192, eff=1408, experts=8, identity=8, top=2, shared=2816, layers=4, batch=16),
             dict(name='w3072_h32x64_kv8_m12x64x256_e12x1024_L4', width=3072, heads=32, kv=8, dim=64, window=512, keep=128, mh=12,
                  mdim=64, mvdim=256, ff=8192, eff=1024, experts=12, identity=4, top=4, shared=2048, layers=4)]
    if getattr(args, 'sizes', None):
        sizes = [sz for i, sz in enumerate(sizes) if str(i) in args.sizes.split(',')]
    vocab, L, CTX_D, NEW_D = 32064, 2048, 2048, 32
    out = []
    for sz in sizes:
        B = sz.get('batch', 4)
        cfg = _dugalix_cfg(sz['width'], sz['heads'], sz['kv'], sz['dim'], sz['window'], sz['keep'], sz['mh'], sz['mdim'], sz['mvdim'],
                           sz['ff'], sz['eff'], sz['experts'], sz['identity'], sz['top'], sz['shared'], sz['layers'], vocab)
        m = DugalixB200(cfg, weights.random_dugalix_weights(cfg, 0, device=dev), dtype=torch.bfloat16)
        _, nums = _engine_model_numbers(m, B, L, CTX_D, NEW_D, vocab, args, hbm, tf)
        row = dict(size=sz['name'], batch=B, prompt=L, dugalix=nums)
        del m
        torch.cuda.empty_cache()
        # Tagenex at equal size: the same attention shape and window in every layer, the same dense unit and experts (gated there)
        att = {'type': 'attention', 'mixer': {'heads': sz['heads'], 'kv_heads': sz['kv'], 'dim': sz['dim'], 'vdim': sz['dim'],
                                              'scale': sz['dim'] ** -0.5, 'v_mix': False, 'mask': {'size': sz['window']}}}
        dense = {'kind': 'dense', 'ff': sz['ff'], 'limit': 7.0}
        mix = {'kind': 'moe', 'expert': {'ff': sz['eff'], 'limit': 7.0}, 'router': {'experts': sz['experts'], 'top': sz['top']}}
        tcfg = {'architecture': 'Tagenex', 'vocab': vocab, 'width': sz['width'], 'norm': {'eps': 1e-5},
                'layers': [dict(att, mlp=(mix if i else dense)) for i in range(sz['layers'])]}
        tm = TagenexB200(tcfg, weights.random_tagenex_weights(tcfg, 0, device=dev), dtype=torch.bfloat16)
        _, row['tagenex_equal_size'] = _engine_model_numbers(tm, B, L, CTX_D, NEW_D, vocab, args, hbm, tf)
        del tm
        torch.cuda.empty_cache()
        out.append(row)
    _emit({"metric": "dugalix_prefill_decode_tok_per_s", 'arch': 'dugalix', 'dtype': 'bf16', 'data': 'synthetic', 'n_gpus': 1,
          'steps': args.steps, 'warmup': max(3, args.warmup), 'peaks': {'hbm_gbs': hbm, 'bf16_tflops': tf}, 'sizes': out})


# ------------------------------------------------------------------------------------------------ --arch danalorn
def _danalorn_cfg(width, heads, kv, dim, lat_dim, lat_rot, rank, q_rank, window, gh, gdim, gvdim, ff, layers, vocab):
    lat = {'type': 'latent_attention',
           'mixer': {'heads': heads, 'dim': lat_dim, 'rot_dim': lat_rot, 'vdim': lat_dim, 'kv_rank': rank, 'q_rank': q_rank,
                     'scale': (lat_dim + lat_rot) ** -0.5, 'mask': {'size': window}, 'rot': {'base': 10000.0, 'dims': lat_rot}}}
    att = {'type': 'attention', 'mixer': {'heads': heads, 'kv_heads': kv, 'dim': dim, 'vdim': dim, 'scale': dim ** -0.5,
                                          'q_temp': {'coef': 0.25, 'every': 128}}}
    gla = {'type': 'gla', 'mixer': {'heads': gh, 'dim': gdim, 'vdim': gvdim, 'tau': 8.0}}
    order = [lat, att, gla, gla]
    return {'architecture': 'Danalorn', 'vocab': vocab, 'width': width, 'norm': {'eps': 1e-5},
            'embedding': {'scale': width ** 0.5, 'bigram': {'buckets': 65521, 'mul_prev': 37, 'mul_cur': 11}},
            'layers': [dict(order[i % 4], mlp={'kind': 'dense', 'ff': ff}) for i in range(layers)]}


def run_danalorn(args):
    """Throughput of the Danalorn design on the continuous-batching engine at layer sizes of a real model (random weights, bf16
    serving mode), beside Dugalix, the closest existing model (same engine, page pool with state rows, sandwich norms, relu^2 units,
    product kernels, attention kernels and a recurrent scan of the same layout), at equal width, depth, attention shape, recurrent
    state shape and feed-forward size. One JSON line: per size the prefill and decode tok/s of both and, per kernel family, time and
    achieved FLOP/s (prefill) or bytes/s (decode) against the measured peaks."""
    import torch
    import phi3_b200  # noqa: F401
    from phi3_b200 import weights
    from phi3_b200.dugalix import DugalixB200
    from phi3_b200.danalorn import DanalornB200
    hbm, _ = peaks()
    tf = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json'))).get('bf16_tflops', 1590.0) if os.path.exists(
        os.path.join(ROOT, 'MEASURED_PEAKS.json')) else 1590.0
    dev = torch.device('cuda:0')
    sizes = [dict(name='w2048_h16x128_kv4_lat(64+32)r96_g8x128x256_ff8192_L4', width=2048, heads=16, kv=4, dim=128, lat_dim=64,
                  lat_rot=32, rank=96, q_rank=768, window=1024, gh=8, gdim=128, gvdim=256, ff=8192, layers=4),
             dict(name='w2048_h16x128_kv4_lat(64+32)r96_g8x128x256_ff8192_L4_b16', width=2048, heads=16, kv=4, dim=128, lat_dim=64,
                  lat_rot=32, rank=96, q_rank=768, window=1024, gh=8, gdim=128, gvdim=256, ff=8192, layers=4, batch=16),
             dict(name='w3072_h32x64_kv8_lat(64+32)r96_g12x64x256_ff8192_L4', width=3072, heads=32, kv=8, dim=64, lat_dim=64,
                  lat_rot=32, rank=96, q_rank=1024, window=512, gh=12, gdim=64, gvdim=256, ff=8192, layers=4)]
    if getattr(args, 'sizes', None):
        sizes = [sz for i, sz in enumerate(sizes) if str(i) in args.sizes.split(',')]
    vocab, L, CTX_D, NEW_D = 32064, 2048, 2048, 32
    out = []
    for sz in sizes:
        B = sz.get('batch', 4)
        cfg = _danalorn_cfg(sz['width'], sz['heads'], sz['kv'], sz['dim'], sz['lat_dim'], sz['lat_rot'], sz['rank'], sz['q_rank'],
                            sz['window'], sz['gh'], sz['gdim'], sz['gvdim'], sz['ff'], sz['layers'], vocab)
        m = DanalornB200(cfg, weights.random_danalorn_weights(cfg, 0, device=dev), dtype=torch.bfloat16)
        _, nums = _engine_model_numbers(m, B, L, CTX_D, NEW_D, vocab, args, hbm, tf)
        row = dict(size=sz['name'], batch=B, prompt=L, danalorn=nums)
        del m
        torch.cuda.empty_cache()
        # Dugalix at equal size: windowed attention of the same shape in every layer, a matrix memory of the recurrent state's shape
        # in every other layer, the same dense unit
        rot = lambda dims, factor=None: {'base': 500000.0, 'dims': dims, **({'scaling': {'factor': factor}} if factor else {})}
        par = {'type': 'parallel',
               'mixer': {'left': {'heads': sz['heads'], 'kv_heads': sz['kv'], 'dim': sz['dim'], 'vdim': sz['dim'], 'scale': sz['dim'] ** -0.5,
                                  'mask': {'size': sz['window'], 'keep_first': 64}, 'rot': rot(sz['dim'], 4.0)},
                         'right': {'heads': sz['gh'], 'dim': sz['gdim'], 'vdim': sz['gvdim'], 'gate_cap': 15.0},
                         'left_scale': 0.7, 'right_scale': 0.7}}
        sig = {'type': 'attention', 'mixer': {'heads': sz['heads'], 'kv_heads': sz['kv'], 'dim': sz['dim'], 'vdim': sz['dim'],
                                              'scale': sz['dim'] ** -0.5, 'mask': {'size': sz['window']}, 'rot': rot(sz['dim'] // 2)}}
        dcfg = {'architecture': 'Dugalix', 'vocab': vocab, 'width': sz['width'], 'norm': {'eps': 1e-5}, 'residual_mult': 0.6,
                'layers': [dict(sig if i % 2 else par, mlp={'kind': 'dense', 'ff': sz['ff']}) for i in range(sz['layers'])]}
        dm = DugalixB200(dcfg, weights.random_dugalix_weights(dcfg, 0, device=dev), dtype=torch.bfloat16)
        _, row['dugalix_equal_size'] = _engine_model_numbers(dm, B, L, CTX_D, NEW_D, vocab, args, hbm, tf)
        del dm
        torch.cuda.empty_cache()
        out.append(row)
    _emit({"metric": "danalorn_prefill_decode_tok_per_s", 'arch': 'danalorn', 'dtype': 'bf16', 'data': 'synthetic', 'n_gpus': 1,
          'steps': args.steps, 'warmup': max(3, args.warmup), 'peaks': {'hbm_gbs': hbm, 'bf16_tflops': tf}, 'sizes': out})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--arch', default='phi3', choices=['phi3', 'tagenex', 'tapalix', 'dugalix', 'danalorn'],
                    help='phi3: the headline workload (default); tagenex / tapalix / dugalix / danalorn: prefill / decode throughput of '
                         'that design on the continuous-batching engine, beside the closest existing model at equal size')
    ap.add_argument('--sizes', default='', help='with --arch dugalix / danalorn: indices of the sizes to run, with commas (default: all)')
    args = ap.parse_args()
    if not (args.gpus > 1 and int(os.environ.get('WORLD_SIZE', 1)) == 1):      # the self-launching parent just relays its child
        _claim_stdout()
    if args.impl == 'reference':
        return run_reference(args)
    if args.arch == 'tagenex':
        return run_tagenex(args)
    if args.arch == 'tapalix':
        return run_tapalix(args)
    if args.arch == 'dugalix':
        return run_dugalix(args)
    if args.arch == 'danalorn':
        return run_danalorn(args)
    world = int(os.environ.get('WORLD_SIZE', 1))
    if args.gpus > 1 and world == 1:
        # convenience: self-launch under torchrun when called directly with --gpus N
        cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={args.gpus}',
               '--master-addr', '127.0.0.1', '--master-port', '29517', os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    run_cuda(args)


if __name__ == '__main__':
    main()

"""Continuous-batching engine: the step function, the sequence table and the scheduler for models that run a ragged token
batch against the shared page pool (paged.PagePool).

The Phi-3 drivers (api._generate) serve one rectangular batch per call: all rows start together and the call ends when the last
row ends. This engine serves a stream of requests instead:

  Engine.step(entries, end)   one model step. `entries` = [(request id, new token ids, indices among them whose logits are
                              wanted)]; a request is admitted at its first entry, may skip steps, and may bring any number of
                              tokens (a prompt portion cut anywhere, or one decoded token). All entries run as ONE batch.
                              `end` = requests whose slot and pages go back to the pool after the step.
  Scheduler                   greedy / nucleus generation on top of step(): admits waiting prompts while slots and pages last,
                              cuts long prompts into portions under a token budget per step, runs the portions beside the
                              single decoded tokens of the running requests, samples on the device with the framework's
                              p3_row_stats / p3_top_p_sample kernels, and frees a request's pages the step it finishes.

A model plugs in with kv_layout(), cache_dtype(), prepare(max_context) and forward(StepBatch, pool) (tagenex.TagenexB200), and
with state_layout() when its layers carry a recurrent state per sequence (dugalix.DugalixB200, danalorn.DanalornB200): the pool then keeps one row of
fp32 numbers per slot and state buffer, and the step's descriptors list the sequences of the step (first row, rows, slot, first
position) for the kernels that walk a sequence's rows in order.
"""
import os

import numpy as np
import torch
from . import _lib
from ._lib import call, ptr
from .paged import PagePool, PoolExhausted, PAGE
from .lm_base import StepBatch



def _stream():
    return torch.cuda.current_stream().cuda_stream


class Engine:
    def __init__(self, model, max_tokens, n_slots=4):
        self.model, self.dev = model, model.dev
        state_layout = model.state_layout() if hasattr(model, 'state_layout') else ()
        self.pool = PagePool(model.kv_layout(), max_tokens, n_slots, model.cache_dtype(), self.dev, state_layout)
        self.stateful = bool(state_layout)                   # recurrent layers: a request's tokens of a step are ONE run of rows
        model.prepare(self.pool.n_pages * PAGE)
        self.q_tile = int(getattr(model, 'q_tile', 32))      # query rows per CTA of the model's prefill attention kernel
        self.slot_of = {}                                    # request id -> slot
        self.steps = 0
        # decode-only steps (every entry brings one token) are captured as CUDA graphs, keyed by what fixes their launches: the
        # number of requests, of wanted rows, and the 128-key bucket of the longest context (it sets the key slices of the decode
        # attention). A key runs eagerly the first time it is seen, is captured the second time and replayed from then on; the
        # step's descriptors are copied into the graph's static buffer before each replay.
        self.use_graphs = os.environ.get('P3_LM_GRAPH', '1') != '0' and self.dev.type == 'cuda'
        self._graphs = {}

    # ------------------------------------------------------------------ sequence table
    def length(self, rid):
        return self.pool.length[self.slot_of[rid]]

    def live(self):
        return list(self.slot_of)

    def finish(self, rid):
        self.pool.release(self.slot_of.pop(rid))

    def can_take(self, rid, n_new):
        """would `n_new` more tokens of request `rid` (known or new) fit right now?"""
        if rid in self.slot_of:
            return self.pool.can_extend(self.slot_of[rid], n_new)
        return bool(self.pool.free_slots) and -(-n_new // PAGE) <= len(self.pool.free_pages)

    # ------------------------------------------------------------------ one step
    def build_batch(self, entries):
        """host side of a step: slots, pages, positions, attention tiles -> one int32 upload"""
        pool = self.pool
        # refuse the whole step before anything is taken if its slots or pages cannot be had
        new_ids = {rid for rid, toks, _ in entries if len(toks) and rid not in self.slot_of}
        if len(new_ids) > len(pool.free_slots):
            raise PoolExhausted(f'{len(new_ids)} new requests but {len(pool.free_slots)} of {pool.n_slots} sequence slots free')
        grow = {}
        for rid, toks, _ in entries:
            grow[rid] = grow.get(rid, 0) + len(toks)
        need = sum(pool.pages_needed(self.slot_of[r], n) if r in self.slot_of else -(-n // PAGE) for r, n in grow.items())
        if need > len(pool.free_pages):
            raise PoolExhausted(f'page pool exhausted: the step wants {need} pages, {len(pool.free_pages)} of {pool.n_pages} free')
        if self.stateful and any(n > 1 for n in (sum(1 for r, t, _ in entries if r == rid and len(t)) for rid in grow)):
            raise ValueError('a request may bring its tokens of a step in one entry only: its recurrent state advances once per step')
        ids, slots, poss, pf, dec, want, seqs = [], [], [], [], [], [], []
        slot_seq = [0] * pool.n_slots                        # slot -> its record in seqs (slots without tokens are never looked up)
        row = 0
        for rid, toks, wanted in entries:
            n = len(toks)
            if n == 0:
                continue
            if rid not in self.slot_of:
                self.slot_of[rid] = pool.admit()
            s = self.slot_of[rid]
            p0 = pool.extend(s, n)
            ids.extend(int(t) for t in toks)
            slots.extend([s] * n)
            poss.extend(range(p0, p0 + n))
            slot_seq[s] = len(seqs)
            seqs.append((row, n, s, p0))
            if n == 1:
                dec.append((row, 1, s, p0))
            else:
                for r0 in range(0, n, self.q_tile):
                    pf.append((row + r0, min(self.q_tile, n - r0), s, p0 + r0))
            for i in wanted:
                if not 0 <= i < n:
                    raise IndexError(f'request {rid}: wanted index {i} outside its {n} tokens')
                want.append(row + i)
            row += n
        T = row
        b = StepBatch()
        b.T, b.n_pf, b.n_dec, b.R, b.n_seq, b.n_slots = T, len(pf), len(dec), len(want), len(seqs), pool.n_slots
        b.max_pos = max(poss) if poss else 0
        if T == 0:
            return b
        flat = np.concatenate([np.asarray(ids, np.int32), np.asarray(slots, np.int32), np.asarray(poss, np.int32),
                               np.asarray(pf, np.int32).reshape(-1), np.asarray(dec, np.int32).reshape(-1),
                               np.asarray(seqs, np.int32).reshape(-1), np.asarray(want, np.int32),
                               np.asarray(slot_seq, np.int32)])
        pad = (-3 * T) % 4                                   # tile records are read as 16-byte vectors
        flat = np.concatenate([flat[:3 * T], np.zeros(pad, np.int32), flat[3 * T:]])
        d = torch.from_numpy(flat).to(self.dev)
        self._bind(b, d)
        pool.sync()
        return b

    @staticmethod
    def _bind(b, d):
        """point the batch's descriptor views into the flat int32 buffer d"""
        T = b.T
        pad = (-3 * T) % 4
        b.flat = d
        b.ids, b.tok_slot, b.tok_pos = d[:T], d[T:2 * T], d[2 * T:3 * T]
        o = 3 * T + pad
        b.pf_tiles = d[o:o + 4 * b.n_pf]
        o += 4 * b.n_pf
        b.dec_tiles = d[o:o + 4 * b.n_dec]
        o += 4 * b.n_dec
        b.seqs = d[o:o + 4 * b.n_seq]                        # {first row, rows, slot, first position} per sequence of the step
        o += 4 * b.n_seq
        b.want_rows = d[o:o + b.R]
        o += b.R
        b.slot_seq = d[o:o + b.n_slots]

    def step(self, entries, end=(), trace=None):
        """-> fp32 logits [number of wanted rows, vocab] on the device (None if nothing is wanted), rows in the order of the
        entries and of their wanted indices"""
        b = self.build_batch(entries)
        if not b.T:
            logits = None
        elif (self.use_graphs and trace is None and b.n_pf == 0 and getattr(self.model, 'profile', None) is None
              and getattr(self.model, 'graph_safe', lambda batch: False)(b)):
            logits = self._graph_step(b)
        else:
            logits = self.model.forward(b, self.pool, trace=trace)
        for rid in end:
            if rid in self.slot_of:
                self.finish(rid)
        self.steps += 1
        return logits


    def _graph_step(self, b):
        from .model import capture_graph
        key = (b.n_dec, b.R, -(-(b.max_pos + 1) // 128))
        ent = self._graphs.get(key)
        if ent is None:
            if len(self._graphs) >= 64:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = {}
            return self.model.forward(b, self.pool)
        if 'graph' not in ent:
            sb = StepBatch()
            sb.T, sb.n_pf, sb.n_dec, sb.R, sb.max_pos = b.T, 0, b.n_dec, b.R, b.max_pos
            sb.n_seq, sb.n_slots = b.n_seq, b.n_slots
            self._bind(sb, torch.empty_like(b.flat))
            sb.flat.copy_(b.flat)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            try:
                with capture_graph(graph):
                    out = self.model.forward(sb, self.pool)
            except Exception:
                # a step that cannot be captured runs eagerly, and so do all later ones (nothing of it has run yet)
                self.use_graphs = False
                self._graphs.clear()
                torch.cuda.synchronize()
                return self.model.forward(b, self.pool)
            ent['graph'], ent['out'], ent['batch'] = graph, out, sb
        else:
            ent['batch'].flat.copy_(b.flat)
        ent['graph'].replay()
        return None if ent['out'] is None else ent['out'].clone()


class _Seq:
    __slots__ = ('rid', 'prompt', 'fed', 'out', 'max_new', 'done')

    def __init__(self, rid, prompt, max_new):
        self.rid, self.prompt, self.fed, self.out, self.max_new, self.done = rid, list(prompt), 0, [], max_new, False


class Scheduler:
    """Generation over Engine.step with continuous batching and chunked prefill.

    token_budget   most tokens one step may run (decoded tokens first, the rest goes to prompt portions)
    chunk          longest prompt portion of one request in one step
    Sampling is greedy (top_p None) or nucleus; both run on the device, one host read of the sampled ids per step."""

    def __init__(self, engine, token_budget=2048, chunk=512, eos_id=None, top_p=None, temperature=1.0, seed=0):
        self.e, self.budget, self.chunk, self.eos = engine, int(token_budget), int(chunk), eos_id
        self.top_p, self.temperature = top_p, float(temperature)
        self.gen = torch.Generator(device=engine.dev).manual_seed(int(seed))
        self.waiting, self.running = [], []
        self._next = 0

    def add(self, prompt, max_new):
        if len(prompt) == 0:
            raise ValueError('empty prompt')
        if -(-(len(prompt) + max_new) // PAGE) > self.e.pool.n_pages:
            raise PoolExhausted(f'a request of {len(prompt)} + {max_new} tokens can never fit the page pool')
        s = _Seq(self._next, prompt, int(max_new))
        self._next += 1
        self.waiting.append(s)
        return s

    def _sample(self, logits):
        R, V = logits.shape
        tok = torch.empty(R, dtype=torch.int32, device=logits.device)
        if self.top_p is None:
            call('p3_row_stats', ptr(logits), R, logits.stride(0), V, ptr(tok), None, None, 0, None, None, 0, None, None, _stream())
        else:
            u = torch.rand(R, generator=self.gen, device=logits.device)
            call('p3_top_p_sample', ptr(logits), R, logits.stride(0), V, float(self.top_p), self.temperature, ptr(u), ptr(tok),
                 None, None, 0, _stream())
        return tok.tolist()

    def step(self):
        """plan one batch, run it, sample; returns the sequences that finished in this step"""
        e = self.e
        entries, samplers, budget = [], [], self.budget
        reserved = 0                                          # pages promised to earlier entries of this step
        free = len(e.pool.free_pages)

        def pages_for(s, n):
            return e.pool.pages_needed(e.slot_of[s.rid], n) if s.rid in e.slot_of else -(-n // PAGE)

        for s in self.running:                                # running requests first: one decoded token or the next portion
            if budget <= 0:
                break
            if s.fed < len(s.prompt):
                n = min(self.chunk, len(s.prompt) - s.fed, budget)
                toks = s.prompt[s.fed:s.fed + n]
            else:
                n, toks = 1, [s.out[-1]]
            need = pages_for(s, n)
            if reserved + need > free:
                continue                                      # waits for pages that a finishing request will give back
            reserved += need
            last = s.fed + n >= len(s.prompt)
            entries.append((s.rid, toks, [n - 1] if last else []))
            if last:
                samplers.append(s)
            s.fed += n
            budget -= n
        while self.waiting and budget > 0 and len(e.slot_of) + sum(1 for x in entries if x[0] not in e.slot_of) < e.pool.n_slots:
            s = self.waiting[0]
            n = min(self.chunk, len(s.prompt), budget)
            # admit only if the whole request can still get its pages (no preemption in this scheduler)
            total = -(-(len(s.prompt) + s.max_new) // PAGE)
            held = sum(-(-(len(r.prompt) + r.max_new) // PAGE) for r in self.running)
            if held + total > e.pool.n_pages:
                break
            self.waiting.pop(0)
            self.running.append(s)
            reserved += -(-n // PAGE)
            last = n >= len(s.prompt)
            entries.append((s.rid, s.prompt[:n], [n - 1] if last else []))
            if last:
                samplers.append(s)
            s.fed = n
            budget -= n
        if not entries:
            if self.running or self.waiting:
                raise PoolExhausted('no request can make progress: the page pool is too small for the running set')
            return []
        logits = e.step(entries)
        finished = []
        if samplers:
            toks = self._sample(logits)
            for s, t in zip(samplers, toks):
                s.out.append(int(t))
                if len(s.out) >= s.max_new or (self.eos is not None and t == self.eos):
                    s.done = True
        for s in [s for s in self.running if s.done]:
            self.running.remove(s)
            e.finish(s.rid)
            finished.append(s)
        return finished

    def run(self):
        done = []
        while self.running or self.waiting:
            done.extend(self.step())
        return sorted(done, key=lambda s: s.rid)


def generate_tokens(model, prompts, max_new=32, max_tokens=None, n_slots=4, eos_id=None, top_p=None, temperature=1.0, seed=0,
                    token_budget=2048, chunk=512):
    """prompts: list of token-id lists -> list of generated id lists (greedy unless top_p is given). The pool holds `max_tokens`
    tokens (default: enough for n_slots of the longest request)."""
    if max_tokens is None:
        longest = max(len(p) for p in prompts) + max_new
        max_tokens = n_slots * (-(-longest // PAGE) * PAGE)
    sch = Scheduler(Engine(model, max_tokens, n_slots), token_budget, chunk, eos_id, top_p, temperature, seed)
    seqs = [sch.add(p, max_new) for p in prompts]
    sch.run()
    return [s.out for s in seqs]

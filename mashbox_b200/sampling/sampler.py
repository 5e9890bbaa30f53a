"""Picks the next token of each row on the device and brings the ids to the host once per step.

Rows that are plainly greedy (temperature 0, no penalties) take the argmax kernel (lowest index of the maximum).  Any
other row takes the sampling kernel: penalties -> temperature -> top_k -> top_p -> min_p -> one Gumbel-max draw, with
random bits from Philox keyed by (seed, index of the token in the row's answer), so a row redraws the same tokens when
it is batched differently or recomputed after a preemption.  Penalty state (counts of generated tokens, the set of
prompt + generated tokens) lives per state slot and is made only when a request asks for a penalty.
"""
import numpy as np
import torch

from .. import ops as kernels

ROW = np.dtype([("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("rep", "<f4"), ("freq", "<f4"),
                ("pres", "<f4"), ("top_k", "<i4"), ("slot", "<i4"), ("seed_lo", "<u4"), ("seed_hi", "<u4"),
                ("step", "<i4"), ("logits_row", "<i4")])


class Sampler:
    def __init__(self, vocab, max_slots, device):
        self.V, self.max_slots, self.device = int(vocab), int(max_slots), device
        self.cnt = self.seen = None
        self.work = None
        self.ret = self.host = None

    def _penalty_state(self):
        if self.cnt is None:
            self.cnt = torch.zeros((self.max_slots, self.V), dtype=torch.int32, device=self.device)
            self.seen = torch.zeros((self.max_slots, self.V), dtype=torch.uint8, device=self.device)

    def start_row(self, slot, prompt, generated):
        """Rebuilds the penalty state of one slot from the request's tokens (at its first token, and again when a
        preempted request has been recomputed)."""
        self._penalty_state()
        self.cnt[slot].zero_()
        self.seen[slot].zero_()
        toks = torch.tensor(list(prompt) + list(generated), dtype=torch.int32).to(self.device)
        kernels.penalty_fill(self.cnt[slot], self.seen[slot], toks, len(prompt), len(prompt) + len(generated), self.V)

    def sample(self, logits, rows, err=None):
        """logits (R, V) float32 on the device; rows: [(SamplingParams, token index, state slot or -1)], one per row of
        logits in order.  -> list of token ids (one device-to-host copy)."""
        return self.wait(self.sample_async(logits, rows, err))

    @staticmethod
    def pack(rows):
        """The rows' settings as the kernels read them (one ROW each), as an int32 array; None when every row is plainly
        greedy (the argmax kernel needs none)."""
        if all(p.plain_greedy for p, _, _ in rows):
            return None
        packed = np.zeros(len(rows), ROW)
        for i, (p, step, slot) in enumerate(rows):
            packed[i] = (p.temperature, p.top_p, p.min_p, p.repetition_penalty, p.frequency_penalty,
                         p.presence_penalty, p.top_k, slot if p.penalised else -1, p.seed & 0xFFFFFFFF,
                         (p.seed >> 32) & 0xFFFFFFFF, step, i)
        return packed.view(np.int32)

    def sample_async(self, logits, rows, err=None, params=None, trace=False):
        """Launches the sampling kernels and starts the copy of the ids (and of the kernels' error word, when given)
        to pinned host memory.  -> a handle for wait().  params: pack(rows) already on the device (the engine sends it
        with the step's arrays; a copy from pageable memory here would make the host wait for the GPU).  trace: the
        hash of every row's logits and the gap between its two largest travel with the ids (trace_of())."""
        n = len(rows)
        if n == 0:
            return None
        if self.ret is None or self.ret.shape[0] < 3 * n + 1:
            cap = 3 * max(n, self.max_slots) + 1            # ids | error word | (hash, gap) per row
            self.ret = torch.empty(cap, dtype=torch.int32, device=self.device)
            self.host = [torch.empty(cap, dtype=torch.int32).pin_memory() for _ in range(2)]
            self.turn = 0
        out = self.ret[:n]
        if all(p.plain_greedy for p, _, _ in rows):
            kernels.argmax(logits[:n], out)
        else:
            if params is None:
                params = torch.from_numpy(self.pack(rows)).to(self.device)
            if any(p.penalised for p, _, _ in rows):
                self._penalty_state()
            if self.work is None or self.work.shape[0] < n:
                self.work = torch.empty((max(n, self.max_slots), self.V), dtype=torch.float32, device=self.device)
            cuts = any(p.temperature > 0 and (p.top_k > 0 or p.top_p < 1.0 or p.min_p > 0.0) for p, _, _ in rows)
            kernels.sample(logits, self.work, params, self.cnt, self.seen, n, out, any_cut=cuts, keep_work=False)
        if err is not None:
            self.ret[n:n + 1].copy_(err)
        size = n + 1
        if trace:
            kernels.logit_trace(logits[:n], self.ret[n + 1:3 * n + 1].view(n, 2))
            size = 3 * n + 1
        self.turn ^= 1
        host = self.host[self.turn]
        host[:size].copy_(self.ret[:size], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return host, n, ev, err, trace

    @staticmethod
    def trace_of(pending):
        """-> [(hash, gap)] per row of a step sampled with trace=True, after wait()"""
        host, n, _, _, trace = pending
        return kernels.read_logit_trace(host[n + 1:3 * n + 1].numpy()) if trace else None

    def wait(self, pending):
        """-> the token ids of sample_async (raises when a kernel of the step left an error code)"""
        if pending is None:
            return []
        host, n, ev, err, _ = pending
        ev.synchronize()
        vals = host[:n + 1].tolist()
        if err is not None and vals[n]:
            err.zero_()
            raise kernels.KernelError("a kernel reported: " + kernels.DEVICE_ERRORS.get(vals[n], f"code {vals[n]}"))
        return vals[:n]

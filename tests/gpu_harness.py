"""Plumbing for the GPU tests of single kernels: a paged cache laid out by hand (pages in shuffled order) and the
descriptors the attention kernels read."""
import numpy as np
import torch

from tests.plain import llama as plain

DEV = "cuda:0"


def to_dev(a, dtype=None):
    t = torch.as_tensor(np.asarray(a)) if not isinstance(a, torch.Tensor) else a
    return t.to(DEV if dtype is None else DEV, dtype) if dtype is not None else t.to(DEV)


def i32(a):
    return torch.as_tensor(np.asarray(a, np.int32)).to(DEV)


class PagedSequences:
    """S sequences of given lengths with random (or given) keys and values, stored in pages in a shuffled order.
    The last q_len[s] positions of each sequence are the step's queries."""

    def __init__(self, lengths, q_lens, H, KV, HD, page, dtype, seed=0, extra_pages=3, rows=None):
        g = torch.Generator().manual_seed(seed)
        self.lengths, self.q_lens, self.H, self.KV, self.HD, self.page, self.dtype = lengths, q_lens, H, KV, HD, page, dtype
        S = len(lengths)
        self.q = [torch.randn(n, H, HD, generator=g) for n in lengths]
        self.k = [torch.randn(n, KV, HD, generator=g) for n in lengths]
        self.v = [torch.randn(n, KV, HD, generator=g) for n in lengths]
        self.rows = list(range(S)) if rows is None else rows           # block-table row of each sequence
        self.max_blocks = max(-(-n // page) for n in lengths) + 1
        self.num_pages = sum(-(-n // page) for n in lengths) + extra_pages
        self.perm = torch.randperm(self.num_pages, generator=g).tolist()

    def round(self):
        """values as the device holds them"""
        r = (lambda t: t.to(self.dtype).float())
        self.q, self.k, self.v = [r(t) for t in self.q], [r(t) for t in self.k], [r(t) for t in self.v]
        return self

    def build(self):
        S, page, KV, HD = len(self.lengths), self.page, self.KV, self.HD
        n_rows = max(self.rows) + 1
        table = np.full((n_rows, self.max_blocks), -1, np.int32)
        kpool = torch.full((self.num_pages, KV, page, HD), float("nan"))
        vpool = torch.full((self.num_pages, KV, page, HD), float("nan"))
        nxt = 0
        for s, n in enumerate(self.lengths):
            for b in range(-(-n // page)):
                pg = self.perm[nxt]
                nxt += 1
                table[self.rows[s], b] = pg
                lo, hi = b * page, min(n, (b + 1) * page)
                kpool[pg, :, :hi - lo] = self.k[s][lo:hi].transpose(0, 1)
                vpool[pg, :, :hi - lo] = self.v[s][lo:hi].transpose(0, 1)
        # slots never written stay NaN in float32 pools so that a read past a sequence's end shows; bf16 gets zeros
        if self.dtype != torch.float32:
            kpool, vpool = torch.nan_to_num(kpool, nan=0.0), torch.nan_to_num(vpool, nan=0.0)
        self.table = i32(table)
        self.kpool, self.vpool = kpool.to(DEV, self.dtype).contiguous(), vpool.to(DEV, self.dtype).contiguous()
        q_start = np.concatenate([[0], np.cumsum(self.q_lens)[:-1]])
        self.q_start, self.q_len = i32(q_start), i32(self.q_lens)
        self.pos0 = i32([n - q for n, q in zip(self.lengths, self.q_lens)])
        self.seq_row = i32(self.rows)
        self.positions = i32(np.concatenate([np.arange(n - q, n) for n, q in zip(self.lengths, self.q_lens)]))
        self.tok_row = i32(np.repeat(self.rows, self.q_lens))
        self.N = int(sum(self.q_lens))
        qs = torch.cat([self.q[s][n - q:] for s, (n, q) in enumerate(zip(self.lengths, self.q_lens))])
        self.q_dev = qs.reshape(self.N, self.H * HD).to(DEV, self.dtype).contiguous()
        return self

    def reference(self, scale, window=None):
        """plain attention over each whole sequence, the query rows of the step only -> (N, H * HD) float64"""
        out = []
        for s, (n, ql) in enumerate(zip(self.lengths, self.q_lens)):
            o = plain.attention(self.q[s].double(), self.k[s].double(), self.v[s].double(), scale, window=window)
            out.append(o[n - ql:])
        return torch.cat(out)


def mma_items(seqs, G, target_splits=1, decode_rows=16, prefill_rows=64, split_prefill=True):
    """work lists of the tensor-core kernel: every sequence with at most decode_rows packed rows goes to the decode
    form, the others to the prompt form; sequences of at most 16 tokens are cut into target_splits splits"""
    dec, pre, part_base, part_tok = [], [], [], []
    q_start = np.concatenate([[0], np.cumsum(seqs.q_lens)[:-1]])
    for s, ql in enumerate(seqs.q_lens):
        rows = ql * G
        decode = rows <= decode_rows
        tiles = 1 if decode else -(-rows // prefill_rows)
        ns = target_splits if ql <= 16 and (decode or split_prefill) else 1
        if ns > 1:
            part_base.append(len(part_tok) // 2)
            for t in range(ql):
                part_tok += [int(q_start[s]) + t, ns]
        else:
            part_base.append(-1)
        for m in range(tiles):
            for sp in range(ns):
                (dec if decode else pre).append((s, m, sp, ns))
    return dec, pre, part_base, part_tok

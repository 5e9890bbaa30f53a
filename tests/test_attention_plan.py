"""The attention mixer's work list (parts/attention.py: prepare, many_splits), on the CPU with a stand-in for the step
context and for the kernels' capability queries: whatever the batch, every decode sequence is covered by its splits
exactly once, clusters are only chosen when the device holds all of them at once, and crowded batches are cut by the
model of partly filled rounds."""
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from mashbox_b200.parts.attention import Attention, KEY_TILE, many_splits

# what one B200 answers for the decode form at head size 128: clusters of c blocks it holds at once
ACTIVE = {2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33}


class FakeOps:
    def attention_mma_supports(self, HD): return True
    def attention_tc5_supports(self, HD, page): return True
    def attention_tc5_rows(self): return 256
    def attention_tma_supports(self, HD, page): return True
    def attention_tma_max_cluster(self, HD): return 8
    def attention_tma_active_clusters(self, HD, c): return ACTIVE[c]


class Inputs(dict):
    def add(self, name, array):
        self[name] = np.asarray(array)


def plan(lengths, new, options=None, heads=32, kv=8, window=None):
    att = Attention(hidden=heads * 128, heads=heads, kv_heads=kv, head_dim=128, window=window)
    q_start = np.concatenate([[0], np.cumsum(new)[:-1]]).tolist()
    ctx = SimpleNamespace(options=dict(options or {}), memo={}, S=len(lengths), q_len=list(new), q_start=q_start,
                          pos0=[n - q for n, q in zip(lengths, new)], dtype=torch.bfloat16, ops=FakeOps(),
                          cache=SimpleNamespace(page_size=16), inputs=Inputs())
    att.prepare(ctx)
    p = ctx.memo[att.plan_key()]
    dec = ctx.inputs[p["name"] + "dec"].reshape(-1, 4)
    pre = ctx.inputs[p["name"] + "pre"].reshape(-1, 4)
    return p, dec, pre, ctx.inputs[p["name"] + "part_base"], ctx.inputs[p["name"] + "part_tok"].reshape(-1, 2)


def check_cover(p, dec, pre, part_base, part_tok, lengths, new, G=4):
    seen = {}
    for s, m, sp, ns in list(dec) + list(pre):
        seen.setdefault((s, m), []).append((sp, ns))
    for s, (n, q) in enumerate(zip(lengths, new)):
        tiles = [k for k in seen if k[0] == s]
        assert tiles, f"sequence {s} has no block"
        for k in tiles:
            ns = seen[k][0][1]
            assert sorted(sp for sp, _ in seen[k]) == list(range(ns)) and all(x == ns for _, x in seen[k])
            assert ns <= max(1, -(-n // KEY_TILE) // 2) or ns == 1 or p["cluster"]
            assert (part_base[s] >= 0) == (ns > 1 and not (p["cluster"] and q * G <= 16))
    if p["cluster"]:
        c = p["cluster"]
        assert len(dec) % c == 0
        for i in range(0, len(dec), c):                               # a cluster is the splits of one sequence, in order
            assert [tuple(r) for r in dec[i:i + c]] == [(dec[i][0], 0, sp, c) for sp in range(c)]
    # the partial buffers: one place per token of a split sequence
    assert len(part_tok) == sum(q for s, q in enumerate(new) if part_base[s] >= 0)


@pytest.mark.parametrize("batch,keys", [(1, 8192), (2, 8192), (3, 8192), (4, 8192), (5, 8192), (8, 8192), (11, 8192),
                                        (16, 8192), (18, 8192), (20, 8192), (24, 8192), (40, 8192), (48, 8192),
                                        (64, 8192), (8, 100), (4, 131072)])
def test_decode_batches(batch, keys):
    lengths, new = [keys] * batch, [1] * batch
    p, dec, pre, part_base, part_tok = plan(lengths, new)
    check_cover(p, dec, pre, part_base, part_tok, lengths, new)
    assert len(pre) == 0
    base = batch * 8
    if p["cluster"]:
        assert base <= ACTIVE[p["cluster"]]                         # all clusters of the launch on the device at once
    if batch == 4 and keys == 8192:
        assert p["cluster"] == 7                                      # 32 clusters: 33 of 8 would be a full house
    if batch in (1, 2) and keys == 8192:
        assert not p["cluster"] and dec[0][3] == (32 if batch == 1 else 16)
    if batch == 20 and keys == 8192:
        assert not p["cluster"] and dec[0][3] == 3                   # 480 blocks: no thin last round
    if batch in (24, 64) and keys == 8192:
        assert dec[0][3] == 1
    if batch == 40 and keys == 8192:
        assert dec[0][3] == 4


def test_random_batches_are_covered():
    rng = random.Random(5)
    for _ in range(200):
        S = rng.randint(1, 40)
        lengths = [rng.choice([1, 2, 63, 64, 65, 500, 4096, 20000]) for _ in range(S)]
        new = [min(n, rng.choice([1, 1, 1, 2, 4, 5, 64, 700])) for n in lengths]
        window = rng.choice([None, None, 128, 1000])
        opts = rng.choice([{}, {"attention_clusters": False}, {"attention_prefill_kernel": "mma"}, {"attention_kernel": "mma"}])
        p, dec, pre, part_base, part_tok = plan(lengths, new, opts, window=window)
        check_cover(p, dec, pre, part_base, part_tok, lengths, new)
        if p["cluster"]:
            n_decode = sum(1 for q in new if q * 4 <= 16)
            assert n_decode * 8 <= ACTIVE[p["cluster"]] and len(dec) == n_decode * p["cluster"]


def test_many_splits_model():
    # one round that fills the device, or less: nothing to gain
    assert many_splits(256, 256 * 128, 296, 128) == 1
    assert many_splits(192, 192 * 128, 296, 128) == 1
    # a thin second round (320 blocks on 296 places) is the worst case: cut further
    assert many_splits(320, 320 * 128, 296, 128) == 4
    assert many_splits(160, 160 * 128, 296, 128) == 3
    assert many_splits(384, 384 * 128, 296, 128) in (2, 3)          # measured within 1.3 % of each other
    # short sequences: a block's own start and finish, and the meeting of the splits, outweigh a thin round
    assert many_splits(160, 160 * 32, 296, 128) == 1
    assert many_splits(192, 192 * 16, 296, 128) == 1
    # never more than asked for, never fewer than one
    for blocks in range(1, 1200, 7):
        for most in (1, 2, 4):
            assert 1 <= many_splits(blocks, blocks * 50, 296, 128, most) <= most
            assert 1 <= many_splits(blocks, blocks * 50, 444, 64, most) <= most

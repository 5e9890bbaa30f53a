"""The attention mixer: grouped-query attention over the paged cache.

q = h Wq^T (+bq), k, v likewise from one fused product (the three weights are concatenated at load); q and k are
rotated, k and v written to the layer's pages, then every query attends to the cached keys of its own sequence up to
its own position -- the step's own tokens are read from the cache like the older ones, so a portion of a prompt, a
single decoded token and a whole prompt all take the same path.  Query head h reads kv head h // (H / KV); scores are
scaled by head_dim^-0.5 (or `scale`), softmax and the weighted sum are float32; `window` w limits a query to the last w
positions.  Formulas: src/mashbox/gguf/archs/dense.py:339-348, src/mashbox/runtime/attention.py:54-93.

Kernels: the float32 path, and head sizes the tensor-core kernel does not take, use the plain paged kernel (one warp
per token and head, fixed order).  The bf16 path packs the G query heads of a kv head into the rows of an MMA tile and
runs the flash kernel: row tiles of 64 for prompt portions, tiles of 16 with the keys split over warps (and over
blocks, merged by a second kernel) for decode tokens.  `prepare` builds that work list on the host.
"""
import numpy as np

from ..cache.manager import CacheNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .base import PartSpec, make, register

DECODE_ROWS, PREFILL_ROWS, KEY_TILE = 16, 64, 64


def many_splits(blocks, work, slots, head_dim, most=4):
    """Into how many splits (1 to `most`) to cut each of `blocks` decode-form tiles of the TMA attention kernel, `work`
    key tiles in all, when there are more of them than half the `slots` the device has for such blocks.  The model: the
    blocks run in rounds of `slots`; a round of n blocks of w key tiles takes the longer of what the memory needs for
    them (n w tiles at 6.5 TB/s, but never less than `enough` blocks' worth: that many blocks, with three or four
    stages of 64 keys in flight each, about 19 MB, keep the memory busy) and what one block needs for itself (7 us to
    start, meet and finish, half a microsecond a tile); splits cost 4 us and 0.15 us each on top (their partial
    results meet through global memory).  The fewest splits within 1 % of the best."""
    tile_bytes = 2 * 64 * head_dim * 2
    enough = max(1, int(19.2e6 // ((3 if head_dim > 64 else 4) * tile_bytes)))
    tile_us = tile_bytes / 6.5e6                                 # a tile's share of the memory's time
    costs = []
    for ns in range(1, max(1, most) + 1):
        n, w = blocks * ns, work / (blocks * ns)
        full, rest = divmod(n, slots)
        alone = 7.0 + 0.5 * w                                     # a block by itself
        t = full * max(slots * w * tile_us, alone)
        if rest:
            t += max(max(rest, enough) * w * tile_us, alone)
        costs.append(t + (4.0 + 0.15 * ns if ns > 1 else 0.0))
    best = min(costs)
    return 1 + next(i for i, c in enumerate(costs) if c <= 1.01 * best)


class Attention:
    @property
    def graph_safe(self):
        """forward() depends on the batch only through the lengths of the step's arrays; so must the position encoding"""
        return self.position is None or bool(getattr(self.position, "graph_safe", False))

    def __init__(self, hidden, heads, kv_heads, head_dim, bias=False, position=None, window=None, scale=None,
                 prefix="", names=None):
        self.D, self.H, self.KV, self.HD = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.H % self.KV:
            raise ConfigError(f"{heads} heads do not divide into {kv_heads} kv heads")
        self.bias, self.window = bool(bias), (int(window) if window else None)
        self.scale = float(scale) if scale else self.HD ** -0.5
        self.prefix = prefix
        n = dict(q="attn_q", k="attn_k", v="attn_v", o="attn_output")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.position = make("position", position) if isinstance(position, PartSpec) else position
        self.wqkv = self.bqkv = self.wo = self.bo = None

    # ------------------------------------------------------------------------------------------ weights
    def wants(self):
        H, KV, HD, D = self.H, self.KV, self.HD, self.D
        shapes = dict(q=(H * HD, D), k=(KV * HD, D), v=(KV * HD, D), o=(D, H * HD))
        w = [Want(self.names[r] + ".weight", shapes[r], "matrix") for r in "qkvo"]
        if self.bias:
            w += [Want(self.names[r] + ".bias", (shapes[r][0],), "vector") for r in "qkvo"]
        return w + (self.position.wants() if self.position is not None else [])

    def bind(self, tensors, env):
        import torch
        t = lambda r, s: tensors[self.names[r] + s]
        self.wqkv = torch.cat([t("q", ".weight"), t("k", ".weight"), t("v", ".weight")], 0).contiguous()
        self.wo = t("o", ".weight")
        if self.bias:
            self.bqkv = torch.cat([t("q", ".bias"), t("k", ".bias"), t("v", ".bias")], 0).contiguous()
            self.bo = t("o", ".bias")
        if self.position is not None:
            self.position.bind(tensors, env)

    def cache_need(self):
        return CacheNeed.keys_and_values(self.KV, self.HD, self.window)

    def state_need(self):
        return None

    # ------------------------------------------------------------------------------------------ planning
    def uses_mma(self, ctx):
        import torch
        return ctx.dtype == torch.bfloat16 and ctx.ops.attention_mma_supports(self.HD) and not ctx.options.get(
            "plain_attention", False)

    def uses_tc5(self, ctx):
        """prompt-form tiles go to the tcgen05 kernel (its own number of packed rows per block, no splits) when it takes
        the sizes"""
        return (ctx.options.get("attention_prefill_kernel", "tc5") == "tc5"
                and ctx.ops.attention_tc5_supports(self.HD, ctx.cache.page_size))

    def plan_key(self):
        # everything the work list depends on: the head size decides the kernel and its rows per tile
        return ("attention", self.H // self.KV, self.KV, self.HD, self.window)

    def prepare(self, ctx):
        """Work list of the flash kernel for this step: (sequence, row tile, split, splits) per block, decode-form
        sequences (at most 16 packed rows) and prompt-form ones apart; sequences cut into splits get a place in the
        partial buffers."""
        if not self.uses_mma(ctx):
            return
        key = self.plan_key()
        if key in ctx.memo:
            return
        G, KV = self.H // self.KV, self.KV
        target = int(ctx.options.get("attention_target_blocks", 296))
        max_splits = int(ctx.options.get("attention_max_splits", 32))
        S = ctx.S
        tc5 = self.uses_tc5(ctx)
        pre_rows = ctx.ops.attention_tc5_rows() if tc5 else PREFILL_ROWS
        decode_form = [ctx.q_len[s] * G <= DECODE_ROWS for s in range(S)]
        tiles = [1 if decode_form[s] else -(-ctx.q_len[s] * G // pre_rows) for s in range(S)]
        # the two forms are two launches: each is cut into splits by its own number of blocks
        base = {f: max(1, sum(t for t, d in zip(tiles, decode_form) if d == f) * KV) for f in (True, False)}
        dec, pre, part_base, part_tok = [], [], [-1] * S, []

        def key_tiles(s):
            hi = ctx.pos0[s] + ctx.q_len[s]
            lo = max(0, ctx.pos0[s] - self.window + 1) if self.window else 0
            return -(-(hi - lo // KEY_TILE * KEY_TILE) // KEY_TILE)

        # Decode-form sequences on the TMA kernel: when they can all be cut into the same number of splits (set by the
        # longest of them; a shorter one leaves some of its splits empty) the blocks of a sequence and kv head are
        # launched as one thread-block cluster and their results meet in shared memory.
        cluster = 0
        page = ctx.cache.page_size
        if (any(decode_form) and base[True] < target and ctx.options.get("attention_kernel", "tma") == "tma"
                and ctx.ops.attention_tma_supports(self.HD, page) and ctx.options.get("attention_clusters", True)):
            raw = min(max_splits, -(-target // base[True]), max(key_tiles(s) for s in range(S) if decode_form[s]) // 2)
            want = 1 << (max(1, raw).bit_length() - 1)
            # only when the cluster holds all the splits the launch wants anyway: at one or two sequences (32 and 16
            # splits) more, smaller blocks that meet through global memory are faster than clusters of 8
            most = ctx.ops.attention_tma_max_cluster(self.HD)
            longest = max(key_tiles(s) for s in range(S) if decode_form[s])
            if want > most and longest <= 6 * most:
                # ... unless the sequences are short: up to six key tiles per block, the cheaper meeting of a cluster
                # outweighs the longer blocks (one sequence of 2,048 keys: 9.2 us in a cluster of 8, 10.4 as 16 splits)
                raw = want = most
            if 2 <= want <= most:
                # the largest cluster, of any size, that leaves all clusters of the launch on the device at once with
                # room to spare: the kernel before this one still holds SMs when the first clusters are placed
                room = float(ctx.options.get("attention_cluster_room", 0.91))
                fits = [c for c in range(2, min(raw, most) + 1)
                        if base[True] <= room * ctx.ops.attention_tma_active_clusters(self.HD, c)]
                cluster = max(fits) if fits else 0
        if ctx.options.get("attention_cluster_size") is not None and any(decode_form):
            cluster = int(ctx.options["attention_cluster_size"])
        # More decode-form tiles than half the blocks the device holds: cutting them to fill `target` blocks would mean
        # one or two splits, and what then decides is the last, partly filled round of blocks: too few blocks to keep
        # the memory busy (8 kv heads, 8,192 keys: 20 sequences as 320 blocks take 8.2 ms a step, as 480 blocks 6.9; 40
        # as 320 blocks 12.4, as 1,280 10.6).  many_splits() picks the number of splits by a model of that.
        crowd = 0
        if (not cluster and any(decode_form) and ctx.options.get("attention_kernel", "tma") == "tma"
                and ctx.ops.attention_tma_supports(self.HD, page) and ctx.options.get("attention_splits") is None):
            slots = 2 * ctx.ops.attention_tma_active_clusters(self.HD, 2)
            if slots and 2 * base[True] > slots:
                work = sum(key_tiles(s) for s in range(S) if decode_form[s]) * KV
                crowd = many_splits(base[True], work, slots, self.HD, min(4, max_splits))
        for s in range(S):
            kv_tiles = key_tiles(s)
            ns = 1
            if cluster and decode_form[s]:
                for sp in range(cluster):
                    dec.append((0, s, 0, sp, cluster))
                continue
            if ctx.q_len[s] <= DECODE_ROWS and base[decode_form[s]] < target and (decode_form[s] or not tc5):
                ns = max(1, min(max_splits, -(-target // base[decode_form[s]]), kv_tiles // 2))
                ns = 1 << (ns.bit_length() - 1)                    # a power of two: few distinct work-list shapes
            if decode_form[s] and (crowd or ctx.options.get("attention_splits") is not None):
                ns = max(1, min(crowd or int(ctx.options["attention_splits"]), kv_tiles // 2))
            if ns > 1:
                part_base[s] = len(part_tok) // 2
                for t in range(ctx.q_len[s]):
                    part_tok += [ctx.q_start[s] + t, ns]
            dst = dec if decode_form[s] else pre
            for m in range(tiles[s]):
                for sp in range(ns):
                    dst.append((-(ctx.pos0[s] + (m + 1) * pre_rows // G), s, m, sp, ns))
        pre.sort()                                                  # the tiles with the most keys first
        name = "attn%d_" % len([k for k in ctx.memo if k[0] == "attention"])
        flat = lambda items: np.asarray([i[1:] for i in items], np.int32).reshape(-1)
        ctx.inputs.add(name + "dec", flat(dec))
        ctx.inputs.add(name + "pre", flat(pre))
        ctx.inputs.add(name + "part_base", np.asarray(part_base, np.int32))
        ctx.inputs.add(name + "part_tok", np.asarray(part_tok, np.int32))
        ctx.memo[key] = dict(name=name, n_dec=len(dec), n_pre=len(pre), n_part=len(part_tok) // 2,
                             max_splits=max_splits, tc5=tc5, cluster=cluster)

    # ------------------------------------------------------------------------------------------ forward
    fuses_small = True      # forward() takes normed= and residual= (see PreNormBlock)

    def forward(self, ctx, h, run, normed=None, residual=None):
        import torch
        ops, N = ctx.ops, ctx.N
        H, KV, HD = self.H, self.KV, self.HD
        width = (H + 2 * KV) * HD
        qkv = ctx.ws.get("qkv", N, (width,), ctx.dtype)
        group, kpool, vpool = ctx.cache.layer_cache(run.cache)
        table = group.device_table
        page, pages = ctx.cache.page_size, ctx.cache.pool_pages
        rot = self.position.rotation() if self.position is not None else (None, HD, 0)
        # A step in which every sequence brings one token (N == S: that follows from the lengths of the step's arrays):
        # the decode form of the TMA attention kernel rotates, stores and attends in one launch.
        folded = (rot is not None and run.write and N == ctx.S and self.uses_mma(ctx)
                  and ctx.options.get("attention_kernel", "tma") == "tma" and ops.attention_tma_supports(HD, page)
                  and ops.attention_tma_folds_rotation(H // KV) and ctx.options.get("attention_folds_rotation", True)
                  and not (normed is not None and ops.small_qkv_supports(N, self.D)
                           and ctx.options.get("qkv_rope_epilogue", False)))
        if (normed is not None and rot is not None and ops.small_qkv_supports(N, self.D)
                and (ctx.options.get("qkv_rope_epilogue", False) or not folded)):
            # a step of very few tokens: norm, product, rotation and the cache write in one kernel -- where the attention
            # kernel cannot take the rotation in (when it can, it also fetches the cached keys before this product has
            # ended: a one-token step of the 8B shape 3.31 against 3.35 ms)
            x, norm = normed
            w, eps = norm.fusable()
            freqs, rd, pairing = rot
            ops.linear_small_normed_qkv(x, w, eps, self.wqkv, qkv, self.bqkv, ctx.dev("positions"), ctx.dev("tok_row"),
                                        table, kpool if run.write else None, vpool if run.write else None, freqs, H, KV,
                                        HD, rd, pairing, page, pages, ctx.err)
        else:
            if normed is not None:
                x, norm = normed
                w, eps = norm.fusable()
                ops.linear_small_normed(x, w, eps, self.wqkv, qkv, held=ctx.take_held(x, norm))
            else:
                ops.linear(h, self.wqkv, out=qkv)
            freqs, rd, pairing = (None, HD, 0)
            if rot is None:
                if self.bias:
                    raise ConfigError("a position encoding with its own kernel cannot be combined with q/k/v biases")
                self.position.apply(ctx, qkv, H, KV, HD)
            else:
                freqs, rd, pairing = rot
            if not folded:
                ops.rope_kv_write(qkv, self.bqkv, ctx.dev("positions"), ctx.dev("tok_row"), table,
                                  kpool if run.write else None, vpool if run.write else None, freqs, H, KV, HD, rd,
                                  pairing, page, pages, ctx.err)
        out = ctx.ws.get("attn_out", N, (H * HD,), ctx.dtype)
        if self.uses_mma(ctx):
            plan = ctx.memo[self.plan_key()]
            nm = plan["name"]
            n_part, ms = plan["n_part"], plan["max_splits"]
            part_o = part_ml = None
            if n_part:
                part_o = ctx.ws.get("attn_part_o", n_part * H * ms, (HD,), torch.float32, reserve=0)
                part_ml = ctx.ws.get("attn_part_ml", n_part * H * ms, (2,), torch.float32, reserve=0)
            kind = ctx.options.get("attention_kernel", "tma")
            tma = kind == "tma" and ops.attention_tma_supports(HD, page)
            flash = ops.attention_tma if tma else ops.attention_mma
            # the TMA kernel merges the splits itself (the last block of a group does it); the other needs the merge kernel
            fused = (tma and n_part > 0 and ctx.options.get("attention_fused_merge", True)
                     and ops.attention_tma_merges(max(plan["n_pre"], plan["n_dec"]), KV))
            extra = dict(merge=True) if fused else {}
            if folded:
                extra["rope"] = (self.bqkv, freqs, rd, pairing)
            if plan["tc5"] and plan["n_pre"]:
                ops.attention_tc5(qkv, width, out, kpool, vpool, ctx.dev(nm + "pre"), plan["n_pre"], ctx.dev("q_start"),
                                  ctx.dev("q_len"), ctx.dev("pos0"), ctx.dev("seq_row"), table, H, KV, HD, page, pages,
                                  self.window, self.scale, ctx.err)
            for form, n_items, decode in ((nm + "pre", 0 if plan["tc5"] else plan["n_pre"], False),
                                          (nm + "dec", plan["n_dec"], True)):
                if n_items and decode and plan["cluster"]:
                    ops.attention_tma(qkv, width, out, kpool, vpool, ctx.dev(form), n_items, True, ctx.dev("q_start"),
                                      ctx.dev("q_len"), ctx.dev("pos0"), None, ctx.dev("seq_row"), table, None, None, 1,
                                      H, KV, HD, page, pages, self.window, self.scale, ctx.err,
                                      rope=extra.get("rope"), cluster=plan["cluster"])
                elif n_items:
                    flash(qkv, width, out, kpool, vpool, ctx.dev(form), n_items, decode, ctx.dev("q_start"),
                          ctx.dev("q_len"), ctx.dev("pos0"), ctx.dev(nm + "part_base"), ctx.dev("seq_row"),
                          table, part_o, part_ml, ms, H, KV, HD, page, pages, self.window, self.scale, ctx.err, **extra)
            if n_part and not fused:
                ops.attention_merge(part_o, part_ml, ctx.dev(nm + "part_tok"), n_part, out, H, HD, ms)
        else:
            ops.attention_simple(qkv, width, out, ctx.dev("positions"), ctx.dev("tok_row"), table, kpool, vpool, H, KV,
                                 HD, page, pages, self.window, self.scale, ctx.err)
        if residual is not None:
            ctx.add_into_stream(out, self.wo, residual, self.bo)
            return None
        y = ctx.ws.get("delta", N, (self.D,), ctx.dtype)
        ops.linear(out, self.wo, out=y)
        return y, self.bo


register("mixer", "attention", Attention)

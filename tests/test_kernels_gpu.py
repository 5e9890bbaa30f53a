"""-m gpu: every kernel alone against its plain reference, at other sizes than the engine's tiny models: widths and
vocabularies that are no power of two, head sizes in steps of 16, odd head and group counts, several page sizes.  Where
random inputs would hide a fault the inputs are built so that it shows: one far key that takes all the weight, keys on
both sides of a window's edge, pages in shuffled order, pool slots past a sequence's end poisoned."""
import numpy as np
import pytest
import torch

from tests import gpu_harness as G
from tests.plain import llama as plain
from tests.plain import sampling as psamp
from tests.tolerances import KERNEL_BF16, KERNEL_F32, nmse

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    import mashbox_b200.ops as K
    return K


def close(got, want, dtype, what=""):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    tol = (KERNEL_F32 if dtype == torch.float32 else KERNEL_BF16) * float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= tol, f"{what}: max error {err:.3e}, bar {tol:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    K = ops()
    g = torch.Generator().manual_seed(0)
    V, D, N = 1003, 72, 37
    table = torch.randn(V, D, generator=g).to(G.DEV, dtype)
    tok = torch.randint(0, V, (N,), generator=g).int().to(G.DEV)
    x = torch.empty(N, D, device=G.DEV)
    err = K.new_error_word(G.DEV)
    K.embed(tok, table, x, err)
    assert torch.equal(x, table.float()[tok.long()])
    K.check_error_word(err)
    tok[5] = V
    K.embed(tok, table, x, err)
    with pytest.raises(Exception, match="token id outside"):
        K.check_error_word(err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [200, 4096 + 8])
def test_add_rmsnorm(dtype, D):
    K = ops()
    g = torch.Generator().manual_seed(1)
    N, eps = 19, 3e-4
    x0 = torch.randn(N, D, generator=g)
    delta = torch.randn(N, D, generator=g).to(dtype)
    bias, w = torch.randn(D, generator=g), 1 + 0.3 * torch.randn(D, generator=g)
    # no delta
    x = x0.clone().to(G.DEV)
    out = torch.empty(N, D, device=G.DEV, dtype=dtype)
    K.add_rmsnorm(x, None, None, w.to(G.DEV), eps, out)
    close(out, plain.rms_norm(x0.double(), w.double(), eps), dtype, "norm")
    assert torch.equal(x.cpu(), x0)
    # delta + bias, in place
    K.add_rmsnorm(x, delta.to(G.DEV), bias.to(G.DEV), w.to(G.DEV), eps, out)
    v = x0.double() + delta.double() + bias.double()
    close(x, v, torch.float32, "residual sum")
    close(out, plain.rms_norm(v, w.double(), eps), dtype, "add + norm")
    # picked rows: the stream is not written
    x = x0.clone().to(G.DEV)
    rows = torch.tensor([7, 0, 18, 7], dtype=torch.int32, device=G.DEV)
    out4 = torch.empty(4, D, device=G.DEV, dtype=dtype)
    K.add_rmsnorm(x, delta.to(G.DEV), None, w.to(G.DEV), eps, out4, rows)
    v = (x0.double() + delta.double())[rows.long().cpu()]
    close(out4, plain.rms_norm(v, w.double(), eps), dtype, "rows")
    assert torch.equal(x.cpu(), x0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    K = ops()
    g = torch.Generator().manual_seed(2)
    N, F = 13, 333
    gu = (2 * torch.randn(N, 2 * F, generator=g)).to(dtype)
    out = torch.empty(N, F, device=G.DEV, dtype=dtype)
    K.swiglu(gu.to(G.DEV), out)
    a, b = gu[:, :F].double(), gu[:, F:].double()
    close(out, a * torch.sigmoid(a) * b, dtype, "swiglu")


def test_gemm_f32_is_exact_enough_and_does_not_depend_on_the_batch():
    K = ops()
    g = torch.Generator().manual_seed(3)
    N, M, Kd = 70, 130, 77
    a, w = torch.randn(N, Kd, generator=g), torch.randn(M, Kd, generator=g)
    c = K.linear(a.to(G.DEV), w.to(G.DEV))
    close(c, a.double() @ w.double().T, torch.float32, "gemm")
    # the same row alone, in a batch of 3 and in the batch of 70: bit for bit the same
    one = K.linear(a[41:42].to(G.DEV), w.to(G.DEV))
    three = K.linear(a[40:43].to(G.DEV), w.to(G.DEV))
    assert torch.equal(one[0], c[41]) and torch.equal(three[1], c[41])
    # and it is float32 arithmetic, not TF32: a product that TF32 would round away
    a2 = torch.tensor([[1.0, 2.0 ** -12]]), torch.tensor([[1.0, 1.0]])
    assert float(K.linear(a2[0].to(G.DEV), a2[1].to(G.DEV))[0, 0]) == 1.0 + 2.0 ** -12


def test_bf16_product_accumulates_in_float32():
    K = ops()
    g = torch.Generator().manual_seed(4)
    a, w = torch.randn(5, 2048, generator=g).bfloat16(), torch.randn(300, 2048, generator=g).bfloat16()
    c = K.linear(a.to(G.DEV), w.to(G.DEV), out_dtype=torch.float32)
    assert c.dtype == torch.float32
    close(c, a.double() @ w.double().T, torch.float32, "bf16 product, float32 out")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing,HD,RD", [("adjacent", 48, 48), ("adjacent", 32, 16), ("halves", 64, 64), ("halves", 80, 32),
                                           ("adjacent", 20, 12), ("halves", 24, 8), ("halves", 128, 128)])
def test_rope_and_cache_write(dtype, pairing, HD, RD):
    K = ops()
    g = torch.Generator().manual_seed(5)
    H, KV, page = 5, 1 if HD == 48 else 3, 8
    seqs = G.PagedSequences([21, 9, 130], [21, 2, 5], H, KV, HD, page, dtype, seed=6).build()
    N = seqs.N
    qkv = torch.randn(N, (H + 2 * KV) * HD, generator=g).to(dtype)
    bias = 0.5 * torch.randn((H + 2 * KV) * HD, generator=g)
    freqs = plain.rope_frequencies(500000.0, RD, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                                       high_freq_factor=4.0, original_max_position_embeddings=64))
    kpool, vpool = torch.zeros_like(seqs.kpool), torch.zeros_like(seqs.vpool)
    dev = qkv.to(G.DEV).clone()
    err = K.new_error_word(G.DEV)
    K.rope_kv_write(dev, bias.to(G.DEV), seqs.positions, seqs.tok_row, seqs.table, kpool, vpool,
                    torch.from_numpy(freqs).to(G.DEV), H, KV, HD, RD, 0 if pairing == "adjacent" else 1, page,
                    seqs.num_pages, err)
    K.check_error_word(err)
    pos = seqs.positions.cpu().numpy()
    full = qkv.double() + bias.double()
    rope = plain.rope_adjacent if pairing == "adjacent" else plain.rope_halves
    q = rope(full[:, :H * HD].reshape(N, H, HD), pos, freqs)
    k = rope(full[:, H * HD:(H + KV) * HD].reshape(N, KV, HD), pos, freqs)
    v = full[:, (H + KV) * HD:].reshape(N, KV, HD)
    close(dev[:, :H * HD], q.reshape(N, -1), dtype, "rotated q")
    table = seqs.table.cpu().numpy()
    rows = seqs.tok_row.cpu().numpy()
    got_k = torch.stack([kpool[table[r, p // page], :, p % page] for r, p in zip(rows, pos)])
    got_v = torch.stack([vpool[table[r, p // page], :, p % page] for r, p in zip(rows, pos)])
    close(got_k, k, dtype, "k in its pages")
    close(got_v, v, dtype, "v in its pages")
    # nothing else in the pools was touched
    touched = torch.zeros(seqs.num_pages, page, dtype=torch.bool)
    for r, p in zip(rows, pos):
        touched[table[r, p // page], p % page] = True
    assert float(kpool.float().abs().sum(dim=(1, 3)).cpu()[~touched].sum()) == 0.0
    # q only (a layer that reads another layer's cache)
    dev2 = qkv.to(G.DEV).clone()
    K.rope_kv_write(dev2, bias.to(G.DEV), seqs.positions, seqs.tok_row, seqs.table, None, None,
                    torch.from_numpy(freqs).to(G.DEV), H, KV, HD, RD, 0 if pairing == "adjacent" else 1, page,
                    seqs.num_pages, err)
    assert torch.equal(dev2[:, :H * HD], dev[:, :H * HD])
    # a position without a page is reported, not written
    bad = seqs.table.clone()
    bad[seqs.rows[1]] = -1
    K.rope_kv_write(qkv.to(G.DEV).clone(), None, seqs.positions, seqs.tok_row, bad, kpool, vpool, None, H, KV, HD, RD,
                    0, page, seqs.num_pages, err)
    with pytest.raises(Exception, match="block table does not hold"):
        K.check_error_word(err)


def dominant_key(seqs, s, key, head_group=None, gain=40.0):
    """makes key `key` of sequence s take all the weight for that sequence's last query: q_last and k[key] are aligned
    and long, so exp(score) dwarfs every other key"""
    HD = seqs.HD
    d = torch.ones(HD) / HD ** 0.5
    seqs.q[s][-1] = gain * d
    seqs.k[s][key] = gain * d


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("HD,H,KV,page,window", [(48, 6, 2, 8, None), (16, 3, 3, 4, 37), (64, 8, 1, 16, None),
                                                 (256, 2, 1, 16, 100)])
def test_attention_plain_kernel(dtype, HD, H, KV, page, window):
    K = ops()
    lengths, q_lens = [300, 45, 1, 77], [1, 45, 1, 13]
    seqs = G.PagedSequences(lengths, q_lens, H, KV, HD, page, dtype, seed=7, rows=[2, 0, 5, 3])
    dominant_key(seqs, 0, 3 if window is None else 300 - window)      # far away / the window's first key
    seqs.round().build()
    out = torch.empty(seqs.N, H * HD, device=G.DEV, dtype=dtype)
    err = K.new_error_word(G.DEV)
    scale = HD ** -0.5
    K.attention_simple(seqs.q_dev, H * HD, out, seqs.positions, seqs.tok_row, seqs.table, seqs.kpool, seqs.vpool, H, KV,
                       HD, page, seqs.num_pages, window, scale, err)
    K.check_error_word(err)
    close(out, seqs.reference(scale, window), dtype, "plain paged attention")
    far = 3 if window is None else 300 - window
    want = seqs.v[0][far].repeat_interleave(H // KV, 0).reshape(-1).double()
    assert float((out[0].double().cpu() - want).abs().max()) < 0.05 * float(want.abs().max()) + 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_plain_kernel_window_edge(dtype):
    """the key just outside the window must not count, however large its score"""
    K = ops()
    H, KV, HD, page, window = 4, 2, 32, 8, 20
    seqs = G.PagedSequences([90], [1], H, KV, HD, page, dtype, seed=8)
    dominant_key(seqs, 0, 90 - window - 1)                            # one position too old
    seqs.round().build()
    out = torch.empty(1, H * HD, device=G.DEV, dtype=dtype)
    err = K.new_error_word(G.DEV)
    K.attention_simple(seqs.q_dev, H * HD, out, seqs.positions, seqs.tok_row, seqs.table, seqs.kpool, seqs.vpool, H, KV,
                       HD, page, seqs.num_pages, window, HD ** -0.5, err)
    close(out, seqs.reference(HD ** -0.5, window), dtype, "window edge")


MMA_CASES = [  # HD, H, KV, page, window, splits
    (256, 8, 4, 16, None, 2), (96, 6, 2, 8, 70, 1), (80, 4, 1, 16, None, 4), (48, 3, 3, 4, None, 1),
    (128, 6, 2, 16, None, 1), (128, 5, 5, 32, 300, 1), (128, 8, 2, 16, None, 1), (128, 8, 2, 16, None, 4), (64, 6, 2, 8, None, 3), (32, 6, 1, 8, 50, 2),
    (16, 4, 2, 4, None, 1), (128, 32, 8, 32, 700, 8), (64, 5, 5, 16, None, 2), (128, 16, 1, 16, None, 2),
    (64, 32, 8, 16, None, 1), (64, 8, 2, 64, 300, 2), (64, 3, 1, 128, None, 1)]


def run_mma(seqs, window, splits, kind="mma"):
    K = ops()
    H, KV, HD, page = seqs.H, seqs.KV, seqs.HD, seqs.page
    flash = K.attention_mma if kind == "mma" else K.attention_tma
    if kind == "tc5" and not K.attention_tma_supports(HD, page):        # decode-form items beside the tcgen05 kernel:
        flash = K.attention_mma                                        # the kernel the mixer would pick for them
    Gq = H // KV
    dec, pre, part_base, part_tok = G.mma_items(seqs, Gq, splits, prefill_rows=K.attention_tc5_rows() if kind == "tc5" else 64,
                                                split_prefill=kind != "tc5")
    out = torch.full((seqs.N, H * HD), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    err = K.new_error_word(G.DEV)
    n_part = len(part_tok) // 2
    ms = max(splits, 1)
    part_o = torch.full((max(1, n_part) * H * ms, HD), float("nan"), device=G.DEV)
    part_ml = torch.full((max(1, n_part) * H * ms, 2), float("nan"), device=G.DEV)
    if kind == "tc5" and pre:        # prompt-form tiles on tcgen05; decode-form items stay on the TMA kernel
        K.attention_tc5(seqs.q_dev, H * HD, out, seqs.kpool, seqs.vpool, G.i32(np.asarray(pre).reshape(-1)), len(pre),
                        seqs.q_start, seqs.q_len, seqs.pos0, seqs.seq_row, seqs.table, H, KV, HD, page, seqs.num_pages,
                        window, HD ** -0.5, err)
        pre = []
    extra = dict(merge=True) if kind == "tma-merging" else {}
    for items, decode in ((pre, False), (dec, True)):
        if items:
            flash(seqs.q_dev, H * HD, out, seqs.kpool, seqs.vpool, G.i32(np.asarray(items).reshape(-1)),
                  len(items), decode, seqs.q_start, seqs.q_len, seqs.pos0, G.i32(part_base), seqs.seq_row,
                  seqs.table, part_o, part_ml, ms, H, KV, HD, page, seqs.num_pages, window, HD ** -0.5, err, **extra)
    if n_part and not extra:
        K.attention_merge(part_o, part_ml, G.i32(part_tok), n_part, out, H, HD, ms)
    K.check_error_word(err)
    return out


@pytest.mark.parametrize("kind", ["mma", "tma", "tma-merging", "tc5"])
@pytest.mark.parametrize("HD,H,KV,page,window,splits", MMA_CASES)
def test_attention_tensor_core_kernel(HD, H, KV, page, window, splits, kind):
    """prompt portions (one starting at position 0, one in the middle of a long context), single decode tokens with
    short and long contexts and a few tokens at once, in one launch pair; one far key that takes all the weight"""
    lengths, q_lens = [900, 150, 1, 333, 70, 260], [1, 150, 1, 3, 33, 100]
    seqs = G.PagedSequences(lengths, q_lens, H, KV, HD, page, torch.bfloat16, seed=9, rows=[4, 1, 0, 6, 2, 3])
    far = 5 if window is None else 900 - window
    dominant_key(seqs, 0, far)
    seqs.round().build()
    if kind == "tc5" and not ops().attention_tc5_supports(HD, page):
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128 only")
    if kind.startswith("tma") and not ops().attention_tma_supports(HD, page):
        with pytest.raises(Exception, match="does not take these sizes"):
            run_mma(seqs, window, splits, kind)
        return
    out = run_mma(seqs, window, splits, kind)
    close(out, seqs.reference(HD ** -0.5, window), torch.bfloat16, "tensor-core paged attention")
    want = seqs.v[0][far].repeat_interleave(H // KV, 0).reshape(-1).double()
    assert float((out[0].double().cpu() - want).abs().max()) < 0.05 * float(want.abs().max()) + 1e-2


@pytest.mark.parametrize("kind,HD", [("mma", 64), ("tma", 64), ("tma", 128), ("tma-merging", 128), ("tc5", 128),
                                     ("tc5", 64)])
@pytest.mark.parametrize("splits", [1, 4])
def test_attention_tensor_core_kernel_window_edge(splits, kind, HD):
    H, KV, page, window = 8, 2, 16, 130
    seqs = G.PagedSequences([700, 700], [1, 40], H, KV, HD, page, torch.bfloat16, seed=10)
    dominant_key(seqs, 0, 700 - window - 1)                           # one position too old: must not count
    dominant_key(seqs, 1, 700 - window)                               # the first key of the last query's window
    seqs.round().build()
    out = run_mma(seqs, window, splits, kind)
    close(out, seqs.reference(HD ** -0.5, window), torch.bfloat16, "window edge")


def test_attention_kernel_refuses_head_sizes_it_does_not_take():
    K = ops()
    assert [K.attention_mma_supports(h) for h in (16, 32, 48, 64, 96, 128, 256, 8, 40, 272)] == [True] * 7 + [False] * 3
    seqs = G.PagedSequences([20], [1], 2, 1, 40, 8, torch.bfloat16).round().build()
    with pytest.raises(Exception, match="does not take these sizes"):
        run_mma(seqs, None, 1)
    big = G.PagedSequences([20], [1], 1, 1, 512, 8, torch.float32).build()
    out = torch.empty(1, 512, device=G.DEV)
    with pytest.raises(Exception, match="does not take these sizes"):
        K.attention_simple(big.q_dev, 512, out, big.positions, big.tok_row, big.table, big.kpool, big.vpool, 1, 1, 512,
                           8, big.num_pages, None, 1.0, K.new_error_word(G.DEV))


# ------------------------------------------------------------------------------------------------ sampling
def sample_rows(logits, rows, cnt=None, seen=None):
    K = ops()
    from mashbox_b200.sampling.sampler import ROW
    n, V = len(rows), logits.shape[1]
    packed = np.zeros(n, ROW)
    for i, r in enumerate(rows):
        packed[i] = (r.get("temperature", 0.0), r.get("top_p", 1.0), r.get("min_p", 0.0), r.get("rep", 1.0),
                     r.get("freq", 0.0), r.get("pres", 0.0), r.get("top_k", 0), r.get("slot", -1),
                     r.get("seed", 0) & 0xFFFFFFFF, (r.get("seed", 0) >> 32) & 0xFFFFFFFF, r.get("step", 0),
                     r.get("row", i))
    assert K.sample_params_size() == ROW.itemsize
    work = torch.empty(n, V, device=G.DEV)
    out = torch.empty(n, dtype=torch.int32, device=G.DEV)
    K.sample(logits, work, torch.from_numpy(packed.view(np.uint8).copy()).to(G.DEV), cnt, seen, n, out)
    return out.tolist(), work.cpu().numpy()


def test_argmax_takes_the_lowest_index_of_the_maximum():
    K = ops()
    V = 128256 + 3
    lg = torch.zeros(3, V)
    lg[0, [70000, 9, 100000]] = 5.0
    lg[1, V - 1] = 1.0
    lg[2] = -torch.arange(V).float()
    out = torch.empty(3, dtype=torch.int32, device=G.DEV)
    K.argmax(lg.to(G.DEV), out)
    assert out.tolist() == [9, V - 1, 0]
    toks, _ = sample_rows(lg.to(G.DEV), [dict(), dict(), dict()])
    assert toks == [9, V - 1, 0]


def test_cuts_keep_exactly_the_allowed_set_ties_included():
    g = torch.Generator().manual_seed(11)
    V = 509
    lg = (3 * torch.randn(6, V, generator=g)).round(decimals=1)          # rounded: many ties
    rows = [dict(temperature=0.7, top_k=5), dict(temperature=1.3, top_p=0.8), dict(temperature=1.0, min_p=0.05),
            dict(temperature=0.9, top_k=40, top_p=0.7, min_p=0.02), dict(temperature=2.0, top_k=1),
            dict(temperature=1.0, top_p=1e-6)]
    toks, work = sample_rows(lg.to(G.DEV), rows)
    for i, r in enumerate(rows):
        want = psamp.transform(lg[i].numpy(), r["temperature"], r.get("top_k", 0), r.get("top_p", 1.0), r.get("min_p", 0.0))
        kept, want_kept = work[i] > -np.inf, want > -np.inf
        assert (kept == want_kept).all(), (i, kept.sum(), want_kept.sum())
        assert np.allclose(work[i][kept], want[kept], rtol=1e-6)
        assert kept[toks[i]]
    assert (work[4] > -np.inf).sum() == (lg[4] == lg[4].max()).sum()      # top_k 1 keeps the maximum and its ties


@pytest.mark.parametrize("kind", ["peaked", "flat", "ties"])
def test_three_kernel_sampler_equals_the_one_kernel_sampler_at_a_large_vocabulary(kind):
    """the serving path (thresholds found among gathered candidates, draw over chunks) against the kernel that bisects
    whole rows, at the vocabulary of the 8B model: the same kept sets and the same tokens.  Peaked rows take the
    candidate path, flat rows have more candidates than fit and fall back, rows of few distinct values are all ties."""
    K = ops()
    from mashbox_b200.sampling.sampler import ROW
    g = torch.Generator().manual_seed(31)
    V = 128256
    if kind == "peaked":
        lg = torch.randn(8, V, generator=g)
        lg[:, :500] += 6.0 * torch.rand(8, 500, generator=g) + 4.0
    elif kind == "flat":
        lg = 0.5 * torch.randn(8, V, generator=g)
    else:
        lg = torch.randint(0, 4, (8, V), generator=g).float()
    rows = [dict(temperature=0.8, top_p=0.9, seed=1), dict(temperature=1.0, top_k=40, seed=2),
            dict(temperature=0.7, top_k=50, top_p=0.8, min_p=0.01, seed=3), dict(temperature=1.2, min_p=0.05, seed=4),
            dict(temperature=0.9, seed=5), dict(), dict(temperature=0.6, top_p=0.3, seed=7),
            dict(temperature=1.0, top_k=2000, top_p=0.95, seed=8)]
    packed = np.zeros(8, ROW)
    for i, r in enumerate(rows):
        packed[i] = (r.get("temperature", 0.0), r.get("top_p", 1.0), r.get("min_p", 0.0), 1.0, 0.0, 0.0, r.get("top_k", 0), -1,
                     r.get("seed", 0), 0, 3, i)
    params = torch.from_numpy(packed.view(np.uint8).copy()).to(G.DEV)
    dev = lg.to(G.DEV)
    w1, w2 = torch.empty(8, V, device=G.DEV), torch.empty(8, V, device=G.DEV)
    o1, o2 = torch.empty(8, dtype=torch.int32, device=G.DEV), torch.empty(8, dtype=torch.int32, device=G.DEV)
    K.sample(dev, w1, params, None, None, 8, o1)
    K.sample_one_kernel(dev, w2, params, None, None, 8, o2)
    a, b = w1.cpu().numpy(), w2.cpu().numpy()
    for i in range(8):
        if rows[i].get("temperature", 0.0) > 0:
            assert ((a[i] > -np.inf) == (b[i] > -np.inf)).all(), (kind, i, (a[i] > -np.inf).sum(), (b[i] > -np.inf).sum())
            assert 0 < (a[i] > -np.inf).sum()
    assert o1.tolist() == o2.tolist()
    o3 = torch.empty(8, dtype=torch.int32, device=G.DEV)
    K.sample(dev, w1, params, None, None, 8, o3, any_cut=True, keep_work=False)
    assert o3.tolist() == o1.tolist()


def test_draws_equal_the_plain_generator_and_depend_on_seed_and_token_index_only():
    g = torch.Generator().manual_seed(12)
    V = 300
    lg = 2 * torch.randn(1, V, generator=g)
    rows = [dict(temperature=0.8, seed=7, step=s, row=0) for s in range(12)] + \
           [dict(temperature=0.8, seed=(1 << 40) + 7, step=3, row=0)]
    toks, _ = sample_rows(lg.to(G.DEV), rows)
    want = [psamp.sample(lg[0].numpy(), temperature=0.8, seed=r["seed"], step=r["step"]) for r in rows]
    assert toks == want
    assert len(set(toks[:12])) > 3
    # the same row among other rows, in another place of the batch: the same token
    other = 2 * torch.randn(3, V, generator=g)
    both = torch.cat([other, lg]).to(G.DEV)
    toks2, _ = sample_rows(both, [dict(temperature=1.5, seed=1, step=0, row=0), dict(row=1),
                                  dict(temperature=0.8, seed=7, step=5, row=3), dict(temperature=0.3, seed=9, row=2)])
    assert toks2[2] == toks[5]


def test_penalties_and_their_state():
    K = ops()
    V = 200
    g = torch.Generator().manual_seed(13)
    lg = 2 * torch.randn(2, V, generator=g)
    cnt = torch.zeros(4, V, dtype=torch.int32, device=G.DEV)
    seen = torch.zeros(4, V, dtype=torch.uint8, device=G.DEV)
    prompt, generated = [5, 9, 5, 77], [9, 9, 120]
    toks = torch.tensor(prompt + generated, dtype=torch.int32, device=G.DEV)
    K.penalty_fill(cnt[2], seen[2], toks, len(prompt), len(prompt) + len(generated), V)
    c, s = np.zeros(V, np.int32), np.zeros(V, bool)
    c[9], c[120] = 2, 1
    s[[5, 9, 77, 120]] = True
    assert (cnt[2].cpu().numpy() == c).all() and (seen[2].cpu().numpy().astype(bool) == s).all()
    lg[0, 9] = lg[0].max() + 0.5                                          # the favourite is a repeated token
    rows = [dict(rep=1.7, freq=0.4, pres=0.3, slot=2, row=0), dict(temperature=0.9, rep=1.2, pres=1.0, slot=2, seed=3, row=1)]
    got, work = sample_rows(lg.to(G.DEV), rows[:1], cnt, seen)
    want = psamp.sample(lg[0].numpy(), rep=1.7, freq=0.4, pres=0.3, cnt=c, seen=s)
    assert got == [want] and want != 9
    assert np.allclose(work[0], psamp.penalise(lg[0].numpy(), c, s, 1.7, 0.4, 0.3), rtol=1e-6)
    c[want] += 1
    s[want] = True
    assert (cnt[2].cpu().numpy() == c).all() and (seen[2].cpu().numpy().astype(bool) == s).all()   # the pick is counted
    got, _ = sample_rows(lg.to(G.DEV), rows[1:], cnt, seen)
    assert got == [psamp.sample(lg[1].numpy(), temperature=0.9, rep=1.2, pres=1.0, seed=3, cnt=c, seen=s)]
    assert int(cnt[0].sum()) == 0 and int(cnt[3].sum()) == 0


@pytest.mark.parametrize("N,M,K", [(1, 4096, 4096), (8, 6144, 4096), (3, 1000, 200), (16, 4096, 14336), (5, 504, 320), (2, 56, 72),
                                   (8, 5000, 520), (3, 14336, 256), (16, 10008, 136), (2, 28672, 264),
                                   # the cuts of few-tile matrices: two and three blocks a tile, tiles of 64 rows
                                   (8, 2048, 8192), (4, 5120, 3072), (16, 2560, 2560), (3, 1024, 4096), (8, 3072, 8192),
                                   (8, 2048, 2048)])
def test_weight_streaming_product(N, M, K):
    """the product for decode batches that streams W by TMA: a block per row tile where that leaves at most a tile per
    SM (tiles of 32, 48, 64, 112 or 128 rows, the last one of a matrix cut short), else equal shares per SM, row tiles
    that blocks share finished by the block that arrives last; called twice so that the self-resetting counters are
    exercised"""
    K_ = ops()
    g = torch.Generator().manual_seed(14)
    a = torch.randn(N, K, generator=g).bfloat16().to(G.DEV)
    w = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16().to(G.DEV)
    want = a.double() @ w.double().T
    for _ in range(2):
        out = torch.full((N, M), float("nan"), device=G.DEV, dtype=torch.bfloat16)
        K_.linear_stream(a, w, out, "plain")
        close(out, want, torch.bfloat16, "weight-streaming product")
    f32 = torch.full((N, M), float("nan"), device=G.DEV)
    K_.linear_stream(a, w, f32, "float")
    close(f32, want, torch.float32, "weight-streaming product, float32 out")
    one = torch.empty(1, M, device=G.DEV, dtype=torch.bfloat16)
    K_.linear_stream(a[N - 1:].contiguous(), w, one, "plain")
    assert torch.equal(one[0], out[N - 1])                 # a row does not depend on the batch it is in
    F = (M // 2) // 8 * 8
    act = torch.full((N, F), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    wgu = torch.cat([w[:F], w[M - F:]]).contiguous()
    K_.linear_stream(a, wgu, act, "swiglu")
    gt = (a.double() @ wgu[:F].double().T).float().bfloat16().double()
    up = (a.double() @ wgu[F:].double().T).float().bfloat16().double()
    close(act, gt * torch.sigmoid(gt) * up, torch.bfloat16, "weight-streaming fused SwiGLU")
    K_.check_error_word(K_.error_word(G.DEV))


@pytest.mark.parametrize("N,M,K", [(128, 256, 64), (2048, 6144, 4096), (300, 1000, 200), (131, 504, 320), (513, 72, 4096)])
def test_tcgen05_product(N, M, K):
    """TMA + tcgen05.mma with the accumulator in tensor memory, against float64; plain, float32 out and fused SwiGLU"""
    K_ = ops()
    g = torch.Generator().manual_seed(15)
    a = torch.randn(N, K, generator=g).bfloat16().to(G.DEV)
    w = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16().to(G.DEV)
    want = a.double() @ w.double().T
    out = torch.full((N, M), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    K_.linear_tc5(a, w, out, "plain")
    close(out, want, torch.bfloat16, "tcgen05 product")
    assert float((out.double() - want).abs().max()) <= 2.0 ** -8 * float(want.abs().max()) + 1e-6       # one bf16 rounding
    f32 = torch.full((N, M), float("nan"), device=G.DEV)
    K_.linear_tc5(a, w, f32, "float")
    close(f32, want, torch.float32, "tcgen05 product, float32 out")
    F = (M // 2) // 8 * 8
    act = torch.full((N, F), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    wgu = torch.cat([w[:F], w[M - F:]]).contiguous()
    K_.linear_tc5(a, wgu, act, "swiglu")
    gt = (a.double() @ wgu[:F].double().T).float().bfloat16().double()
    up = (a.double() @ wgu[F:].double().T).float().bfloat16().double()
    close(act, gt * torch.sigmoid(gt) * up, torch.bfloat16, "tcgen05 fused SwiGLU product")
    # gate values far outside the exponential's range stay finite and right
    big = torch.full((N, F), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    K_.linear_tc5(a, (wgu.float() * 80).bfloat16(), big, "swiglu")
    assert torch.isfinite(big.float()).all()
    K_.check_error_word(K_.error_word(G.DEV))
    with pytest.raises(Exception, match="does not take these sizes"):
        K_.linear_tc5(a[:, :K - 4].contiguous(), w[:, :K - 4].contiguous(), out, "plain")


@pytest.mark.parametrize("N,M,K", [(1, 6144, 4096), (1, 57, 72), (3, 1000, 2504), (2, 64, 8184)])
def test_matrix_vector_product_that_normalises_and_one_that_adds_to_the_stream(N, M, K):
    """the two folded forms of a one-token step: rmsnorm inside the product that follows it, the residual add inside
    the product that ends a sublayer (also through the long-row kernel)"""
    K_ = ops()
    g = torch.Generator().manual_seed(21)
    x = (3.0 * torch.randn(N, K, generator=g)).to(G.DEV)
    nw = (1.0 + 0.2 * torch.randn(K, generator=g)).to(G.DEV)
    w = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16().to(G.DEV)
    eps = 1e-5
    h = (x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * nw.double()).float().bfloat16()
    out = torch.full((N, M), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    K_.linear_gemv_normed(x, nw, eps, w, out, "plain")
    close(out, h.double() @ w.double().T, torch.bfloat16, "normalising matrix-vector product")
    F = M // 2
    act = torch.full((N, F), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    wgu = torch.cat([w[:F], w[M - F:]]).contiguous()
    K_.linear_gemv_normed(x, nw, eps, wgu, act, "swiglu")
    gt = (h.double() @ wgu[:F].double().T).float().bfloat16().double()
    up = (h.double() @ wgu[F:].double().T).float().bfloat16().double()
    close(act, gt * torch.sigmoid(gt) * up, torch.bfloat16, "normalising gate/up product")
    # the same rows as the norm kernel followed by the plain product
    hh = torch.empty(N, K, device=G.DEV, dtype=torch.bfloat16)
    K_.add_rmsnorm(x.clone(), None, None, nw, eps, hh, None)
    two = torch.empty(N, M, device=G.DEV, dtype=torch.bfloat16)
    K_.linear_gemv(hh, w, two, "plain")
    assert float((out.double() - two.double()).abs().max()) <= 2.0 ** -7 * float(two.double().abs().max())
    # adding into the stream: a (N, K) bf16 against W2 (M, K), x2 (N, M) float32, with and without a bias
    a = torch.randn(N, K, generator=g).bfloat16().to(G.DEV)
    x2 = torch.randn(N, M, generator=g).to(G.DEV)
    bias = torch.randn(M, generator=g).to(G.DEV)
    want = x2.double() + a.double() @ w.double().T
    got = x2.clone()
    K_.linear_gemv_residual(a, w, got)
    close(got, want, torch.float32, "residual add in the product")
    got = x2.clone()
    K_.linear_gemv_residual(a, w, got, bias)
    close(got, want + bias.double(), torch.float32, "residual add with a bias")


@pytest.mark.parametrize("pairing,HD,RD,H,KV,bias", [("adjacent", 64, 64, 4, 2, True), ("halves", 32, 16, 3, 1, False),
                                                     ("halves", 128, 128, 2, 2, True), ("adjacent", 48, 32, 2, 1, False)])
def test_qkv_product_with_rotation_and_cache_write_in_its_epilogue(pairing, HD, RD, H, KV, bias):
    """norm + q/k/v product + rotation + cache write as one kernel (one-token steps) leaves exactly what the normalising
    product followed by the rotate-and-store kernel leaves: q in the buffer, k and v in their pages"""
    K_ = ops()
    g = torch.Generator().manual_seed(23)
    D, page = 256, 8
    seqs = G.PagedSequences([37, 5, 90], [1, 1, 1], H, KV, HD, page, torch.bfloat16, seed=6).build()
    N, M = seqs.N, (H + 2 * KV) * HD
    x = (2.0 * torch.randn(N, D, generator=g)).to(G.DEV)
    nw = (1.0 + 0.2 * torch.randn(D, generator=g)).to(G.DEV)
    w = (torch.randn(M, D, generator=g) / D ** 0.5).bfloat16().to(G.DEV)
    b = (0.5 * torch.randn(M, generator=g)).to(G.DEV) if bias else None
    freqs = torch.from_numpy(plain.rope_frequencies(10000.0, RD, None)).to(G.DEV)
    pr = 0 if pairing == "adjacent" else 1
    err = K_.new_error_word(G.DEV)
    k1, v1 = torch.zeros_like(seqs.kpool), torch.zeros_like(seqs.vpool)
    one = torch.zeros(N, M, device=G.DEV, dtype=torch.bfloat16)
    K_.linear_gemv_normed_qkv(x, nw, 1e-5, w, one, b, seqs.positions, seqs.tok_row, seqs.table, k1, v1, freqs, H, KV, HD, RD,
                              pr, page, seqs.num_pages, err)
    k2, v2 = torch.zeros_like(seqs.kpool), torch.zeros_like(seqs.vpool)
    two = torch.empty(N, M, device=G.DEV, dtype=torch.bfloat16)
    K_.linear_gemv_normed(x, nw, 1e-5, w, two, "plain")
    K_.rope_kv_write(two, b, seqs.positions, seqs.tok_row, seqs.table, k2, v2, freqs, H, KV, HD, RD, pr, page,
                     seqs.num_pages, err)
    K_.check_error_word(err)
    assert torch.equal(one[:, :H * HD], two[:, :H * HD])
    assert torch.equal(k1, k2) and torch.equal(v1, v2) and float(k1.float().abs().sum()) > 0
    # without pools nothing is stored, q is the same
    three = torch.zeros(N, M, device=G.DEV, dtype=torch.bfloat16)
    K_.linear_gemv_normed_qkv(x, nw, 1e-5, w, three, b, seqs.positions, seqs.tok_row, seqs.table, None, None, freqs, H, KV,
                              HD, RD, pr, page, seqs.num_pages, err)
    assert torch.equal(three[:, :H * HD], one[:, :H * HD])


@pytest.mark.parametrize("N,M,K", [(8, 6144, 4096), (16, 56, 72), (3, 1000, 2504), (1, 4096, 4096), (5, 264, 14336), (8, 4096, 4096),
                                   (8, 2048, 8192), (4, 3072, 8192), (16, 1024, 4096), (8, 2048, 2048)])
def test_streaming_products_that_add_to_the_stream_and_take_the_norm_in(N, M, K):
    """the folded forms of a step of at most 16 tokens: the product that ends a sublayer adds into the float32 stream and
    leaves what the norm after it needs (sums of squares by 32 columns, rows times the norm's weight in bf16); the
    product after that norm runs on those rows and scales its float sums by 1 / rms.  Tiles of 128, 64 and 32 rows,
    matrices with one block per tile and with shared tiles; called twice, so the counters have reset themselves"""
    K_ = ops()
    g = torch.Generator().manual_seed(31)
    eps = 1e-5
    a = torch.randn(N, K, generator=g).bfloat16().to(G.DEV)
    w = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16().to(G.DEV)
    x2 = (3.0 * torch.randn(N, M, generator=g)).to(G.DEV)
    x2[N - 1] *= 40.0                                      # rows of very different size: each has its own 1 / rms
    bias = torch.randn(M, generator=g).to(G.DEV)
    nw = (1.0 + 0.2 * torch.randn(M, generator=g)).to(G.DEV)
    want = x2.double() + a.double() @ w.double().T
    for b in (None, bias):
        for _ in range(2):
            got = x2.clone()
            K_.linear_stream_residual(a, w, got, b)
            close(got, want if b is None else want + bias.double(), torch.float32, "residual add in the streaming product")
    tiles = (M + 31) // 32
    sums = torch.full((tiles, 16), float("nan"), device=G.DEV)
    scaled = torch.full((N, M), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    x = x2.clone()
    K_.linear_stream_residual(a, w, x, bias, sums, nw, scaled)
    close(x, want + bias.double(), torch.float32, "residual add that also prepares the norm")
    sq = torch.nn.functional.pad(x.double() ** 2, (0, tiles * 32 - M)).reshape(N, tiles, 32).sum(-1).T
    assert float((sums[:, :N].double() - sq).abs().max()) <= 1e-5 * float(sq.max())
    assert float(sums[:, N:].abs().max() if N < 16 else 0.0) == 0.0
    assert torch.equal(scaled, (x * nw).bfloat16())
    # the product after the norm: x (N, M) is now the stream, W2 (M2, M)
    if M % 8:
        return
    for M2 in (136, 4096 if M <= 4096 else 264) + ((6144, 28672) if (N, M) == (8, 4096) else ()):
        w2 = (torch.randn(M2, M, generator=g) / M ** 0.5).bfloat16().to(G.DEV)
        inv = torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps)
        want2 = (scaled.double() @ w2.double().T) * inv
        out = torch.full((N, M2), float("nan"), device=G.DEV, dtype=torch.bfloat16)
        K_.linear_stream(scaled, w2, out, "plain", sums, eps)
        close(out, want2, torch.bfloat16, "streaming product of the normalised stream")
        # against the norm kernel followed by the product: the same up to the rounding of the normalised row
        hh = torch.empty(N, M, device=G.DEV, dtype=torch.bfloat16)
        K_.add_rmsnorm(x.clone(), None, None, nw, eps, hh, None)
        assert nmse(out.double().cpu().numpy(), (hh.double() @ w2.double().T).cpu().numpy()) <= 4.0 * 2.0 ** -18
        one = torch.empty(1, M2, device=G.DEV, dtype=torch.bfloat16)
        K_.linear_stream(scaled[N - 1:].contiguous(), w2, one, "plain",
                         torch.nn.functional.pad(sums[:, N - 1:N], (0, 15)).contiguous(), eps)
        assert torch.equal(one[0], out[N - 1])             # a row does not depend on the batch it is in
        F = (M2 // 2) // 8 * 8
        act = torch.full((N, F), float("nan"), device=G.DEV, dtype=torch.bfloat16)
        wgu = torch.cat([w2[:F], w2[M2 - F:]]).contiguous()
        K_.linear_stream(scaled, wgu, act, "swiglu", sums, eps)
        gt = ((scaled.double() @ wgu[:F].double().T) * inv).float().bfloat16().double()
        up = ((scaled.double() @ wgu[F:].double().T) * inv).float().bfloat16().double()
        close(act, gt * torch.sigmoid(gt) * up, torch.bfloat16, "streaming gate/up product of the normalised stream")
    K_.check_error_word(K_.error_word(G.DEV))


@pytest.mark.parametrize("N,M,K", [(1, 4096, 4096), (4, 6144, 4096), (2, 509, 320), (3, 4096, 14336), (1, 57, 72), (2, 37, 8200)])
def test_matrix_vector_product(N, M, K):
    """at most 4 tokens: one warp per two rows of W, float32 sums; plain, float32 out and fused SwiGLU"""
    K_ = ops()
    g = torch.Generator().manual_seed(16)
    a = torch.randn(N, K, generator=g).bfloat16().to(G.DEV)
    w = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16().to(G.DEV)
    want = a.double() @ w.double().T
    out = torch.full((N, M), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    K_.linear_gemv(a, w, out, "plain")
    close(out, want, torch.bfloat16, "matrix-vector product")
    assert float((out.double() - want).abs().max()) <= 2.0 ** -8 * float(want.abs().max()) + 1e-6
    f32 = torch.full((N, M), float("nan"), device=G.DEV)
    K_.linear_gemv(a, w, f32, "float")
    close(f32, want, torch.float32, "matrix-vector product, float32 out")
    one = torch.empty(1, M, device=G.DEV, dtype=torch.bfloat16)
    K_.linear_gemv(a[N - 1:].contiguous(), w, one, "plain")
    assert torch.equal(one[0], out[N - 1])                          # a token's result does not depend on the batch
    F = M // 2
    act = torch.full((N, F), float("nan"), device=G.DEV, dtype=torch.bfloat16)
    wgu = torch.cat([w[:F], w[M - F:]]).contiguous()
    K_.linear_gemv(a, wgu, act, "swiglu")
    gt = (a.double() @ wgu[:F].double().T).float().bfloat16().double()
    up = (a.double() @ wgu[F:].double().T).float().bfloat16().double()
    close(act, gt * torch.sigmoid(gt) * up, torch.bfloat16, "matrix-vector fused SwiGLU")
    with pytest.raises(Exception, match="does not take these sizes"):
        K_.linear_gemv(torch.zeros(5, K, device=G.DEV, dtype=torch.bfloat16), w, torch.empty(5, M, device=G.DEV, dtype=torch.bfloat16))


@pytest.mark.parametrize("V", [1, 2, 509, 4096, 128256])
def test_logit_trace_hash_and_gap(V):
    """the order-independent hash sum(bits(lg[v]) * (2 v + 1)) mod 2^32 and the float32 gap between the two largest
    logits of every row (src/mashbox/runtime/engine.py:80-89), against numpy: equal, not close"""
    from tests.test_replay_gpu import np_logit_hash
    K, DEV = ops(), G.DEV
    g = torch.Generator().manual_seed(V)
    lg = (4 * torch.randn(5, V, generator=g)).float()
    if V >= 2:
        lg[1, V // 2] = lg[1].max() + 0.75                   # a clear winner
        lg[2, 0] = lg[2, V - 1] = lg[2].max() + 1.0           # two equal maxima, at both ends: gap 0
        lg[3, V - 1] = -0.0                                  # the sign bit of a zero counts in the hash
        lg[4] = -lg[4].abs() - 1.0                           # all negative
    out = torch.empty((5, 2), dtype=torch.int32, device=DEV)
    K.logit_trace(lg.to(DEV), out)
    got = K.read_logit_trace(out)
    want = np_logit_hash(lg.numpy()) if V >= 2 else [(int(np.float32(x).view(np.uint32)), 0.0) for x in lg[:, 0].numpy()]
    assert got == want
    if V >= 2:
        assert got[2][1] == 0.0 and abs(got[1][1] - 0.75) < 1e-5
        flipped = lg.clone()
        flipped[0, V // 3] = torch.nextafter(flipped[0, V // 3], torch.tensor(float("inf")))
        K.logit_trace(flipped.to(DEV), out)
        assert K.read_logit_trace(out)[0][0] != got[0][0]    # one changed bit changes the hash


@pytest.mark.parametrize("HD,H,KV,page,window,splits,pairing,RD,bias", [
    (128, 8, 2, 16, None, 4, 0, 128, False), (128, 32, 8, 16, None, 8, 0, 128, True), (64, 6, 2, 32, 300, 2, 1, 32, True),
    (64, 32, 8, 8, None, 1, 0, 64, False), (128, 16, 1, 64, None, 2, 1, 128, False), (128, 5, 5, 16, 70, 1, 0, 64, True)])
def test_decode_attention_with_the_rotation_folded_in(HD, H, KV, page, window, splits, pairing, RD, bias):
    """one-token sequences: attention_tma(rope=...) on the raw output of the q/k/v product gives the bits of
    rope_kv_write followed by attention_tma, in the outputs and in the pages (a token at the first slot of a page, at
    the last, alone in its sequence, at a tile's edge; with a window; biases; partial rotation; both pairings)"""
    K = ops()
    lengths = [900, 64, 65, 1, 333, 128, 16]
    Gq = H // KV
    seqs = G.PagedSequences(lengths, [1] * len(lengths), H, KV, HD, page, torch.bfloat16, seed=31).round().build()
    g = torch.Generator().manual_seed(5)
    N, width = len(lengths), (H + 2 * KV) * HD
    qkv = torch.randn(N, width, generator=g).to(G.DEV, torch.bfloat16)
    b = (0.3 * torch.randn(width, generator=g)).to(G.DEV) if bias else None
    freqs = torch.from_numpy(plain.rope_frequencies(10000.0, RD, None)).to(G.DEV)
    dec, pre, part_base, part_tok = G.mma_items(seqs, Gq, splits)
    assert not pre
    items = G.i32(np.asarray(dec).reshape(-1))

    def attend(qkv_in, kpool, vpool, rope):
        out = torch.full((N, H * HD), float("nan"), device=G.DEV, dtype=torch.bfloat16)
        err = K.new_error_word(G.DEV)
        ms = max(splits, 1)
        n_part = len(part_tok) // 2
        part_o = torch.full((max(1, n_part) * H * ms, HD), float("nan"), device=G.DEV)
        part_ml = torch.full((max(1, n_part) * H * ms, 2), float("nan"), device=G.DEV)
        K.attention_tma(qkv_in, width, out, kpool, vpool, items, len(dec), True, seqs.q_start, seqs.q_len, seqs.pos0,
                        G.i32(part_base), seqs.seq_row, seqs.table, part_o, part_ml, ms, H, KV, HD, page, seqs.num_pages,
                        window, HD ** -0.5, err, merge=n_part > 0, rope=rope)
        K.check_error_word(err)
        return out

    k1, v1, q1 = seqs.kpool.clone(), seqs.vpool.clone(), qkv.clone()
    err = K.new_error_word(G.DEV)
    K.rope_kv_write(q1, b, seqs.positions, seqs.tok_row, seqs.table, k1, v1, freqs, H, KV, HD, RD, pairing, page,
                    seqs.num_pages, err)
    K.check_error_word(err)
    want = attend(q1, k1, v1, None)
    k2, v2, q2 = seqs.kpool.clone(), seqs.vpool.clone(), qkv.clone()
    got = attend(q2, k2, v2, (b, freqs, RD, pairing))
    assert torch.equal(q2, qkv)                                         # the product's output is left alone
    assert torch.equal(k2, k1) and torch.equal(v2, v1)
    assert not torch.isnan(got.float()).any() and torch.equal(got, want)
    # and the new token's key really took part: attending without it gives something else
    assert not torch.equal(want, attend(q1, seqs.kpool, seqs.vpool, None))


@pytest.mark.parametrize("HD,H,KV,page,window,cluster,rope", [
    (128, 32, 8, 16, None, 8, True), (128, 8, 2, 16, None, 4, False), (64, 6, 2, 32, 300, 8, True),
    (64, 32, 8, 8, None, 2, False), (128, 16, 1, 64, None, 8, False), (128, 5, 5, 16, 70, 2, True),
    (128, 32, 8, 16, None, 7, True), (64, 6, 2, 32, None, 3, False), (128, 8, 2, 16, 300, 5, True), (64, 4, 4, 16, None, 6, True)])
def test_decode_attention_in_clusters(HD, H, KV, page, window, cluster, rope):
    """the decode form launched as thread-block clusters, one block per split of a sequence and kv head, the splits
    meeting in the cluster's shared memory: the same bits as the launch whose splits meet through global memory and a
    ticket, with and without the rotation folded in; sequences shorter than the splits leave splits empty"""
    K = ops()
    if cluster > K.attention_tma_max_cluster(HD):
        pytest.skip(f"this device places clusters of at most {K.attention_tma_max_cluster(HD)} of these blocks")
    lengths = [2100, 64, 65, 1, 333, 128, 900]
    Gq = H // KV
    seqs = G.PagedSequences(lengths, [1] * len(lengths), H, KV, HD, page, torch.bfloat16, seed=33).round().build()
    dominant_key(seqs, 0, 7)
    seqs.round().build()
    g = torch.Generator().manual_seed(6)
    N, width = len(lengths), (H + 2 * KV) * HD
    if rope:
        q_in = torch.randn(N, width, generator=g).to(G.DEV, torch.bfloat16)
        b = (0.3 * torch.randn(width, generator=g)).to(G.DEV)
        freqs = torch.from_numpy(plain.rope_frequencies(10000.0, HD, None)).to(G.DEV)
        extra, stride = dict(rope=(b, freqs, HD, 0)), width
    else:
        q_in, extra, stride = seqs.q_dev, {}, H * HD
    items = G.i32(np.asarray([(s, 0, sp, cluster) for s in range(N) for sp in range(cluster)]).reshape(-1))
    part_base = G.i32(list(range(N)))

    def attend(kpool, vpool, **how):
        out = torch.full((N, H * HD), float("nan"), device=G.DEV, dtype=torch.bfloat16)
        err = K.new_error_word(G.DEV)
        part_o = torch.full((N * H * cluster, HD), float("nan"), device=G.DEV)
        part_ml = torch.full((N * H * cluster, 2), float("nan"), device=G.DEV)
        K.attention_tma(q_in, stride, out, kpool, vpool, items, N * cluster, True, seqs.q_start, seqs.q_len, seqs.pos0,
                        part_base, seqs.seq_row, seqs.table, part_o, part_ml, cluster, H, KV, HD, page, seqs.num_pages,
                        window, HD ** -0.5, err, **how, **extra)
        K.check_error_word(err)
        return out

    k1, v1 = seqs.kpool.clone(), seqs.vpool.clone()
    want = attend(k1, v1, merge=True)
    k2, v2 = seqs.kpool.clone(), seqs.vpool.clone()
    got = attend(k2, v2, cluster=cluster)
    assert not torch.isnan(got.float()).any() and torch.equal(got, want)
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    if not rope:
        close(got, seqs.reference(HD ** -0.5, window), torch.bfloat16, "decode attention in clusters")

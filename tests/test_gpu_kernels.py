"""Each CUDA kernel alone against its plain float32 reference, at sizes other than the
engine's tiny models: widths and vocabularies that are no power of two, head sizes in
steps of 16, several head groupings, page sizes, windows and key splits.  Where random
data would hide a fault (one far key among hundreds, a window's edge, a page's edge) the
inputs are made so that one key dominates and the output must be that key's value."""
import math

import numpy as np
import pytest
import torch

from tests.plain import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from paged_batch_engine_b200.csrc import ops as o
    return o


def bf16_round(t):
    return t.to(torch.bfloat16).float()


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,vocab", [(88, 517), (3584, 1003)])
def test_embedding(dtype, d, vocab):
    torch.manual_seed(0)
    table = torch.randn(vocab, d).to(dtype)
    ids = torch.randint(0, vocab, (37,), dtype=torch.int32)
    ids[0], ids[1] = 0, vocab - 1
    out = torch.empty(37, d, dtype=torch.float32, device=DEV)
    ops().embedding(out, table.to(DEV), ids.to(DEV))
    assert torch.equal(out.cpu(), plain.embedding(ids.tolist(), table.float()))


# ------------------------------------------------------------------ residual add + rmsnorm
@pytest.mark.parametrize("d", [64, 88, 1000, 3584, 5120])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(d, out_dtype):
    torch.manual_seed(d)
    T, eps = 13, 3e-6
    res = torch.randn(T, d) * 3
    delta = (torch.randn(T, d) * 2).to(out_dtype)
    gain = 1 + 0.1 * torch.randn(d)
    r = res.clone().to(DEV)
    out = torch.empty(T, d, dtype=out_dtype, device=DEV)
    ops().add_rmsnorm(r, delta.to(DEV), gain.to(DEV), out, eps)
    x = res + delta.float()
    want = plain.rmsnorm(x, gain, eps)
    assert torch.equal(r.cpu(), x)                          # the sum is exact float32
    tol = 1e-5 if out_dtype == torch.float32 else 0.0
    if out_dtype == torch.float32:
        assert (out.cpu() - want).abs().max() <= 1e-5 * want.abs().max()
    else:
        assert (out.float().cpu() - want).abs().max() <= 2 ** -8 * want.abs().max()
    # no delta: the residual is only normalised
    r2 = res.clone().to(DEV)
    out2 = torch.empty(T, d, dtype=out_dtype, device=DEV)
    ops().add_rmsnorm(r2, None, gain.to(DEV), out2, eps)
    assert torch.equal(r2.cpu(), res)
    assert (out2.float().cpu() - plain.rmsnorm(res, gain, eps)).abs().max() <= 2 ** -8 * want.abs().max()
    # wanted rows only: the residual stays as it was
    rows = torch.tensor([12, 0, 5], dtype=torch.int32)
    r3 = res.clone().to(DEV)
    out3 = torch.empty(3, d, dtype=out_dtype, device=DEV)
    ops().add_rmsnorm(r3, delta.to(DEV), gain.to(DEV), out3, eps, rows=rows.to(DEV))
    assert torch.equal(r3.cpu(), res)
    assert torch.equal(out3.cpu(), out.cpu()[rows.long()])


# ------------------------------------------------------------------ silu * up
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,inter", [(1, 208), (19, 18944), (300, 37)])
def test_silu_mul(dtype, rows, inter):
    torch.manual_seed(1)
    gu = (torch.randn(rows, 2 * inter) * 3).to(dtype)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    ops().silu_mul(gu.to(DEV), out)
    want = plain.swiglu(gu.float()[:, :inter], gu.float()[:, inter:])
    if dtype == torch.float32:
        assert (out.cpu() - want).abs().max() <= 1e-5
    else:
        assert (out.float().cpu() - want).abs().max() <= 2 ** -8 * want.abs().max()


# ------------------------------------------------------------------ rope + bias + cache write
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,hd,rot,inter", [(4, 2, 16, 16, False), (6, 3, 48, 48, False),
                                               (28, 4, 128, 128, False), (5, 1, 32, 16, False),
                                               (3, 3, 32, 32, True)])
def test_rope_bias_cache_write(dtype, H, KV, hd, rot, inter):
    torch.manual_seed(2)
    T, P, pages, theta = 11, 8, 9, 50000.0
    width = (H + 2 * KV) * hd
    qkv = torch.randn(T, width).to(dtype)
    bias = torch.randn(width) * 0.5
    pos = torch.tensor([0, 1, 2, 3, 700, 701, 9, 4095, 64, 65, 66], dtype=torch.int32)
    slots = torch.randperm(pages * P)[:T].to(torch.int32)
    slots[3] = -1                                            # a row that must not be written
    inv = plain.rope_inv_freq(rot, theta)
    kc = torch.full((pages, KV, P, hd), 7.0, dtype=dtype, device=DEV)
    vc = torch.full((pages, KV, P, hd), 7.0, dtype=dtype, device=DEV)
    q = torch.empty(T, H * hd, dtype=dtype, device=DEV)
    ops().rope_kv_write(qkv.to(DEV), bias.to(DEV), q, kc, vc, pos.to(DEV), slots.to(DEV), inv.to(DEV),
                        H, KV, hd, rot, P, interleaved=inter)
    x = qkv.float() + bias
    qf = x[:, :H * hd].view(T, H, hd)
    kf = x[:, H * hd:(H + KV) * hd].view(T, KV, hd)
    vf = x[:, (H + KV) * hd:].view(T, KV, hd)
    rope = plain.rope_interleaved if inter else plain.rope_rotate_half

    def rotate(t):
        return torch.cat([rope(t[..., :rot], pos, theta), t[..., rot:]], dim=-1)
    want_q, want_k = rotate(qf), rotate(kf)
    tol = 2e-5 if dtype == torch.float32 else 2 ** -7
    scale = want_q.abs().max()
    assert (q.float().cpu().view(T, H, hd) - want_q).abs().max() <= tol * scale
    kc, vc = kc.float().cpu(), vc.float().cpu()
    touched = torch.zeros(pages, P, dtype=torch.bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        page, off = s // P, s % P
        touched[page, off] = True
        assert (kc[page, :, off] - want_k[t]).abs().max() <= tol * scale
        assert (vc[page, :, off] - vf[t]).abs().max() <= tol * scale
    untouched = ~touched
    assert (kc.permute(0, 2, 1, 3)[untouched] == 7.0).all()          # nothing else was written
    assert (vc.permute(0, 2, 1, 3)[untouched] == 7.0).all()
    # a layer that reads another layer's cache writes nothing
    kc2 = torch.full((pages, KV, P, hd), 7.0, dtype=dtype, device=DEV)
    ops().rope_kv_write(qkv.to(DEV), bias.to(DEV), q, None, None, pos.to(DEV), None, inv.to(DEV),
                        H, KV, hd, rot, P, interleaved=inter)
    assert (kc2 == 7.0).all()


# ------------------------------------------------------------------ float32 GEMM
@pytest.mark.parametrize("M,N,K", [(1, 33, 50), (7, 64, 64), (130, 517, 88), (65, 100, 1003)])
def test_sgemm_true_float32(M, N, K):
    torch.manual_seed(3)
    x, w, b = torch.randn(M, K), torch.randn(N, K), torch.randn(N)
    out = torch.empty(M, N, device=DEV)
    ops().sgemm_nt(x.to(DEV), w.to(DEV), b.to(DEV), out)
    want = (x.double() @ w.double().t() + b.double())
    err = (out.cpu().double() - want).abs().max().item()
    assert err <= 2e-6 * math.sqrt(K) * 4          # float32 accumulation; TF32 would be ~1e-3
    # bfloat16 storage in and out, float32 arithmetic
    xb = x.to(torch.bfloat16)
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops().sgemm_nt(xb.to(DEV), w.to(DEV), None, outb)
    wantb = xb.double() @ w.double().t()
    assert (outb.cpu().double() - wantb).abs().max() <= 2 ** -8 * wantb.abs().max()


def test_sgemm_rows_do_not_depend_on_the_batch():
    """One summation order for every output, whichever kernel computes it: the weight-streaming
    kernel (up to 16 rows) and the tiled kernels (tiles of 32, 64
    and 128 rows) give bitwise equal rows; K of 333 is no multiple of 4 (scalar copies), 1,100
    spans three K slices with a ragged last one."""
    torch.manual_seed(4)
    for K in (333, 1100):
        x, w, b = torch.randn(150, K, device=DEV), torch.randn(77, K, device=DEV), torch.randn(77, device=DEV)
        full = torch.empty(150, 77, device=DEV)
        ops().sgemm_nt(x, w, b, full)
        for lo, hi in [(0, 1), (3, 10), (20, 36), (64, 129), (100, 130), (90, 150), (149, 150)]:
            part = torch.empty(hi - lo, 77, device=DEV)
            ops().sgemm_nt(x[lo:hi].contiguous(), w, b, part)
            assert torch.equal(part, full[lo:hi]), (K, lo, hi)       # same summation order: bitwise equal


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16, 17, 40, 200])
def test_sgemm_sizes_that_divide_nothing(M):
    """Rows, columns and depths that are multiples of no tile size, through both kernels; the
    large cases have many tasks a warp slot (weight-streaming kernel) and enough tiles for the
    tiled kernel to keep its K slices in one block."""
    torch.manual_seed(M)
    big = [(19000, 4100)] if M <= 16 else [(300, 1030)] + ([(19000, 1100)] if M == 200 else [])
    for N, K in [(1, 7), (33, 516), (130, 36)] + big:
        x, w, b = torch.randn(M, K), torch.randn(N, K), torch.randn(N)
        out = torch.full((M, N), float("nan"), device=DEV)
        ops().sgemm_nt(x.to(DEV), w.to(DEV), b.to(DEV), out)
        want = x.double() @ w.double().t() + b.double()
        assert (out.cpu().double() - want).abs().max().item() <= 2e-6 * math.sqrt(K) * 4, (M, N, K)


# ------------------------------------------------------------------ paged attention
class AttnCase:
    """Requests with a context already in the cache and q_len new rows each; pages handed
    out in a scrambled order; K and V written by indexing."""

    def __init__(self, H, KV, hd, P, window, reqs, dtype, seed=0, kind="simple", num_pages=None):
        from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
        from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
        o = ops()
        g = torch.Generator().manual_seed(seed)
        self.H, self.KV, self.hd, self.P, self.window, self.dtype, self.kind = H, KV, hd, P, window, dtype, kind
        kind_, tile_rows, _ = o.attention_kernel_config(hd, dtype, kind)
        total_pages = num_pages or sum((c + n + P - 1) // P for c, n in reqs) + 3
        m = CacheManager([KVGroupSpec((0,), KV, hd, window)], P, total_pages, max_requests=64, lifo=True)
        # scramble the free list: take all pages and give them back in random order
        m.set_free_order(0, torch.randperm(total_pages, generator=g).tolist())
        self.k_pages = torch.full((total_pages, KV, P, hd), float("nan"), dtype=dtype, device=DEV)
        self.v_pages = torch.full((total_pages, KV, P, hd), float("nan"), dtype=dtype, device=DEV)
        self.seqs, entries = [], []
        for ctx_len, n in reqs:
            h = m.add_request()
            L = ctx_len + n
            assert m.reserve(h, L)
            k = torch.randn(L, KV, hd, generator=g).to(dtype)
            v = torch.randn(L, KV, hd, generator=g).to(dtype)
            q = torch.randn(L, H, hd, generator=g).to(dtype)
            self.seqs.append((q, k, v, ctx_len, n, h))
            entries.append(StepEntry(h, [0] * n))
        self.manager = m
        self._entries = entries
        self.tile_rows = tile_rows

    def write_cache(self):
        m, P = self.manager, self.P
        for q, k, v, ctx_len, n, h in self.seqs:
            table = m.block_table(h)
            for p in range(ctx_len + n):
                self.k_pages[table[p // P], :, p % P] = k[p].to(DEV)
                self.v_pages[table[p // P], :, p % P] = v[p].to(DEV)

    def run(self):
        from paged_batch_engine_b200.engine.batch import StepContext
        o = ops()
        m = self.manager
        for q, k, v, ctx_len, n, h in self.seqs:
            m.commit(h, ctx_len)
        G = self.H // self.KV
        key = (0, G, self.tile_rows, self.window)
        ctx = StepContext(m, self._entries, torch.device(DEV), [key])
        meta = ctx.attention_work(0, G, self.tile_rows, self.window, self.H, self.hd)
        qrows = torch.cat([q[c:c + n] for q, k, v, c, n, h in self.seqs]).reshape(-1, self.H * self.hd)
        out = torch.full_like(qrows, float("nan")).to(DEV)
        o.paged_attention(qrows.to(DEV).contiguous(), self.k_pages, self.v_pages, out, meta, self.H,
                          self.KV, self.hd, self.hd ** -0.5, self.window, self.P, kind=self.kind)
        self.meta = meta
        return out.float().cpu().view(-1, self.H, self.hd)

    def reference(self):
        outs = []
        for q, k, v, ctx_len, n, h in self.seqs:
            o = plain.causal_attention(q.float(), k.float(), v.float(), self.hd ** -0.5, self.window)
            outs.append(o[ctx_len:ctx_len + n])
        return torch.cat(outs)


ATTN_SHAPES = [
    # H, KV, hd, P, window, [(context, new rows)...]
    (4, 2, 16, 16, None, [(0, 5), (0, 17), (0, 33)]),
    (6, 1, 32, 8, None, [(40, 1), (0, 9), (71, 1), (3, 40)]),
    (6, 3, 48, 8, 24, [(0, 50), (30, 1), (23, 2), (100, 7)]),
    (28, 4, 128, 16, None, [(300, 1), (0, 70), (513, 3)]),
    (8, 8, 64, 32, None, [(1000, 1), (255, 2), (256, 1), (257, 1)]),
    (14, 2, 80, 16, 300, [(700, 1), (290, 20), (0, 400)]),
    (5, 5, 256, 16, None, [(20, 3), (600, 1)]),
]


KINDS = [("simple", torch.float32), ("simple", torch.bfloat16), ("mma", torch.bfloat16)]


@pytest.mark.parametrize("kind,dtype", KINDS, ids=lambda v: str(v).replace("torch.", ""))
@pytest.mark.parametrize("shape", ATTN_SHAPES, ids=lambda s: f"H{s[0]}kv{s[1]}hd{s[2]}P{s[3]}w{s[4]}")
def test_paged_attention(shape, kind, dtype):
    H, KV, hd, P, window, reqs = shape
    case = AttnCase(H, KV, hd, P, window, reqs, dtype, seed=hd, kind=kind)
    case.write_cache()
    got, want = case.run(), case.reference()
    assert not torch.isnan(got).any()
    tol = 2e-5 if dtype == torch.float32 else 2 ** -7
    assert (got - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
    if any(c + n > 256 and n * (H // KV) <= 4 * case.tile_rows for c, n in reqs):
        assert case.meta.num_split_rows > 0 and case.meta.max_splits > 1   # the split path ran


@pytest.mark.parametrize("kind,dtype", KINDS, ids=lambda v: str(v).replace("torch.", ""))
def test_attention_one_key_stands_out(kind, dtype):
    """One key among many gets a large score: the output row must be that key's value.
    The special key sits at a page's first and last slot, at a split's edge, at the
    window's first and last key, and just outside the window (then it must NOT win)."""
    H, KV, hd, P = 4, 2, 32, 16
    L = 1030
    for window, specials in [(None, [0, 15, 16, 255, 256, 511, 512, 1023, 1024, 1029]),
                             (100, [1029, 930, 929])]:
        for j in specials:
            case = AttnCase(H, KV, hd, P, window, [(L - 1, 1)], dtype, seed=j, kind=kind)
            q, k, v, c, n, h = case.seqs[0]
            k.mul_(0.05)
            q[L - 1] = 0
            q[L - 1, :, 0] = 40.0
            k[j, :, 0] = 40.0                      # score 1600/sqrt(32) above all others
            case.write_cache()
            got = case.run()[0]
            visible = window is None or j > (L - 1) - window
            for head in range(H):
                is_special = torch.allclose(got[head], v[j, head // 2].float(), atol=2e-2)
                assert is_special == visible, (window, j, head)
            assert (got - case.reference()[0]).abs().max() <= (2e-5 if dtype == torch.float32 else 2e-2)


def test_attention_mma_prompt_tiles_and_mixed_batch():
    """Long prompt portions (many row tiles, rows mode) beside decoded tokens (keys mode) in
    one launch, with the 7-heads-per-kv-head grouping of the 7B shape."""
    case = AttnCase(28, 4, 128, 16, None, [(0, 200), (777, 1), (130, 90), (2047, 1), (64, 5)],
                    torch.bfloat16, seed=3, kind="mma")
    case.write_cache()
    got, want = case.run(), case.reference()
    assert not torch.isnan(got).any()
    assert (got - want).abs().max().item() <= 2 ** -7 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("H,KV,hd,P,window", [(28, 4, 128, 16, None), (6, 3, 48, 8, 40), (4, 2, 16, 16, None),
                                               (5, 5, 256, 16, None)])
def test_attention_mma_many_decoding_requests(H, KV, hd, P, window, monkeypatch):
    """Decoded tokens through the persistent warp-private instance (one warp streams a whole
    key split), which steps of many work items take: its threshold is set to zero here.
    Contexts end on and off tile, split and page edges; a few short prompt portions ride along."""
    from paged_batch_engine_b200.csrc import ops as pbe_ops
    monkeypatch.setattr(pbe_ops, "DECODE_BLOCK_ITEMS_PER_SM", 0)
    ctxs = [0, 1, 15, 16, 17, 63, 64, 255, 256, 257, 300, 511, 512, 513, 700, 31, 33, 1000, 129, 5]
    reqs = [(c, 1) for c in ctxs] + [(90, 2), (0, 12)]
    case = AttnCase(H, KV, hd, P, window, reqs, torch.bfloat16, seed=hd + len(reqs), kind="mma")
    case.write_cache()
    got, want = case.run(), case.reference()
    assert case.meta.kinds & 4 == 0 and case.meta.kinds & 1          # the many-requests path was taken
    assert not torch.isnan(got).any()
    assert (got - want).abs().max().item() <= 2 ** -7 * max(1.0, want.abs().max().item())
    # one key stands out at the last position of a long context, for every request at once
    case2 = AttnCase(H, KV, hd, P, None, [(600 + 7 * i, 1) for i in range(18)], torch.bfloat16, seed=1, kind="mma")
    for i, (q, k, v, c, n, h) in enumerate(case2.seqs):
        j = [0, 15, 16, 255, 256, 599][i % 6]
        k.mul_(0.05)
        q[c] = 0
        q[c, :, 0] = 40.0
        k[j, :, 0] = 40.0
    case2.write_cache()
    got2 = case2.run()
    for i, (q, k, v, c, n, h) in enumerate(case2.seqs):
        j = [0, 15, 16, 255, 256, 599][i % 6]
        for head in range(H):
            assert torch.allclose(got2[i, head], v[j, head // (H // KV)].float(), atol=3e-2), (i, j, head)


TC5_SHAPES = [
    # H, KV, hd, P, window, [(context, new rows)...]
    (28, 4, 128, 16, None, [(0, 300)]),                           # several key tiles, ragged last row tile
    (28, 4, 128, 16, None, [(1500, 64), (300, 1), (0, 70)]),      # key splits, a decoded token beside portions
    (8, 8, 64, 32, None, [(255, 130), (1000, 1), (0, 17)]),       # head size 64, one row per packed row
    (14, 2, 128, 8, 300, [(700, 40), (290, 20), (0, 400)]),       # window, pages of 8
    (6, 3, 64, 128, 200, [(100, 500), (513, 3)]),                 # pages as large as the key tile
    (16, 2, 128, 64, None, [(37, 19), (2000, 2)]),                # 16 rows x 8 heads: the smallest prompt tile
]


@pytest.mark.parametrize("shape", TC5_SHAPES, ids=lambda s: f"H{s[0]}kv{s[1]}hd{s[2]}P{s[3]}w{s[4]}")
def test_paged_attention_tcgen05(shape):
    """Prompt portions on the tcgen05 kernel (free pages hold NaN), decoded tokens beside them."""
    H, KV, hd, P, window, reqs = shape
    case = AttnCase(H, KV, hd, P, window, reqs, torch.bfloat16, seed=hd + P, kind="tc5")
    case.write_cache()
    out = case.run()
    assert ops().tc5_error_flag(DEV) == 0
    ref = case.reference()
    assert torch.isfinite(out).all()
    assert (out - ref).abs().max().item() < 2e-2


def test_attention_tcgen05_far_key_and_window_edge():
    """One key far back gets all the weight (its value must come through exactly); with a
    window that ends one key after it, it must not be seen at all."""
    H, KV, hd, P = 8, 2, 128, 16
    L, n, far = 900, 40, 131
    for window, seen in ((None, True), (L - n - far, False), (L - n - far + 1, True)):
        case = AttnCase(H, KV, hd, P, window, [(L - n, n)], torch.bfloat16, seed=11, kind="tc5")
        q, k, v, ctx_len, _, _ = case.seqs[0]
        k[far] = 0
        k[far, :, 0] = 8.0
        q[ctx_len, :, 0] = 40.0                            # the portion's first row looks at key `far`
        v[far] = 3.0
        case.write_cache()
        out = case.run()
        assert ops().tc5_error_flag(DEV) == 0
        ref = case.reference()
        assert (out - ref).abs().max().item() < 2e-2
        assert ((out[0] - 3.0).abs().max().item() < 2e-2) == seen


def test_attention_ignores_stale_data_in_reused_and_foreign_pages():
    """Pages beyond a request's length and pages of other requests hold NaN or huge
    values: the result must not change."""
    H, KV, hd, P = 6, 3, 48, 8
    for kind, dtype, tol in (("simple", torch.float32, 2e-5), ("mma", torch.bfloat16, 2e-2)):
        case = AttnCase(H, KV, hd, P, None, [(13, 4), (0, 6)], dtype, seed=5, kind=kind)
        case.k_pages.fill_(1e30)
        case.v_pages.fill_(float("nan"))
        case.write_cache()
        got, want = case.run(), case.reference()
        assert not torch.isnan(got).any() and (got - want).abs().max() <= tol


# ------------------------------------------------------------------ sampling
def test_argmax_ties_go_to_the_lowest_id():
    torch.manual_seed(6)
    logits = torch.randn(5, 151937)
    logits[0, 77] = logits[0, 150000] = 50.0
    logits[1, 151936] = 60.0
    logits[2, 0] = 60.0
    logits[3] = 1.25
    out = ops().argmax(logits.to(DEV)).cpu().tolist()
    assert out == [77, 151936, 0, 0, int(torch.argmax(logits[4]))]
    # a view with a row stride (logits of a wider buffer)
    wide = torch.randn(4, 1000, device=DEV)
    assert ops().argmax(wide[:, :517]).cpu().tolist() == torch.argmax(wide[:, :517], dim=1).cpu().tolist()


@pytest.mark.parametrize("vocab", [517, 32003])
def test_sampler_matches_the_reference_algorithm(vocab):
    rng = np.random.default_rng(vocab)
    rows = []
    cases = [(0.8, 0, 1.0), (1.0, 40, 1.0), (0.7, 0, 0.9), (1.3, 50, 0.5), (0.0, 5, 1.0), (1.0, 1, 1.0),
             (0.5, 0, 0.01), (2.0, 0, 1.0), (0.0, 0, 1.0), (1.0, 200, 0.95)]
    us = [0.0, 0.03, 0.31, 0.5, 0.77, 0.93, 0.99999]
    logits = torch.tensor(rng.normal(0, 2.0, size=(len(cases) * len(us), vocab)), dtype=torch.float32)
    logits[:, 11] = logits[:, 400]                 # exact ties inside every row
    logits[3, :] = logits[3, :].round()            # many ties
    t, k, p, u = [], [], [], []
    for c in cases:
        for x in us:
            t.append(c[0]); k.append(c[1]); p.append(c[2]); u.append(x)
    got = ops().sample(logits.to(DEV), torch.tensor(t, dtype=torch.float32, device=DEV),
                       torch.tensor(k, dtype=torch.int32, device=DEV),
                       torch.tensor(p, dtype=torch.float32, device=DEV),
                       torch.tensor(u, dtype=torch.float32, device=DEV)).cpu().tolist()
    mismatches = 0
    for i, tok in enumerate(got):
        want = plain.sample_row(logits[i].tolist(), t[i], k[i], p[i], uniform=u[i])
        if tok == want:
            continue
        # the only admissible difference: the draw sits within 1e-5 of a boundary of the CDF
        iv = plain.sample_cdf_interval(logits[i].tolist(), tok, t[i], k[i], p[i])
        assert iv is not None, (i, tok, want)
        assert iv[0] - 1e-5 <= u[i] <= iv[1] + 1e-5, (i, tok, want, iv, u[i])
        mismatches += 1
    assert mismatches <= 2


@pytest.mark.parametrize("vocab", [1, 2, 33, 1003, 8192, 8193, 152064])
def test_sampler_binned_selection_equals_the_radix_descent(vocab):
    """The kernel's quick way (bins by distance from the maximum, one bin sorted) and its radix
    descent pick the same token: random rows, scaled rows, masks of -inf and of -1e9, rows of
    equal logits (whose one crowded bin sends the quick way to the descent anyway), ties at the
    top, and every combination of temperature, top-k and top-p."""
    g = torch.Generator().manual_seed(vocab)
    settings = [(0.8, 0, 1.0), (1.0, 40, 1.0), (0.7, 0, 0.9), (1.3, 50, 0.5), (0.1, 50, 0.9), (0.0, 5, 1.0),
                (1.0, 1, 1.0), (0.5, 0, 0.01), (5.0, 0, 0.999), (1.0, 3000, 0.95), (1e-3, 0, 1.0), (1.0, 10 ** 6, 0.3)]
    kinds = 8
    n = len(settings) * kinds * 3
    logits = torch.randn(n, vocab, generator=g) * 2.0
    t, k, p = [], [], []
    i = 0
    for st in settings:
        for kind in range(kinds):
            for _ in range(3):
                row = logits[i]
                if kind == 1:
                    row *= 10.0
                elif kind == 2:
                    row *= 0.01
                elif kind == 3:
                    row[torch.rand(vocab, generator=g) < 0.5] = float("-inf")
                elif kind == 4:
                    row[torch.rand(vocab, generator=g) < 0.7] = -1e9
                elif kind == 5:
                    row.fill_(0.25)
                elif kind == 6:
                    row.copy_(row.round())
                elif kind == 7:
                    row[: max(1, vocab // 3)] = row.max() + 1.0       # a third of the row ties for the top
                t.append(st[0]); k.append(st[1]); p.append(st[2])
                i += 1
    u = torch.rand(n, generator=g)
    u[::7] = 0.0
    u[3::11] = 0.99999994
    args = (logits.to(DEV), torch.tensor(t, dtype=torch.float32, device=DEV), torch.tensor(k, dtype=torch.int32, device=DEV),
            torch.tensor(p, dtype=torch.float32, device=DEV), u.to(DEV))
    o = ops()
    try:
        o.sample_set_mode(1)
        slow = o.sample(*args).cpu()
    finally:
        o.sample_set_mode(0)
    # all rows at once (a block a row), and a few rows a call (a cluster of blocks a row when the
    # vocabulary is large)
    for rows_a_call in (n, 60, 30, 16):      # clusters of 1, 2, 4 and 8 blocks a row
        quick = torch.cat([o.sample(*[a[i:i + rows_a_call].contiguous() for a in args]).cpu()
                           for i in range(0, n, rows_a_call)])
        bad = (slow != quick).nonzero().flatten().tolist()
        assert not bad, (rows_a_call, [(j, t[j], k[j], p[j], float(u[j]), int(slow[j]), int(quick[j])) for j in bad[:5]])


def test_sampler_does_not_depend_on_the_batch_and_follows_the_distribution():
    torch.manual_seed(8)
    V, n = 1003, 4000
    row = torch.randn(V) * 1.5
    u = torch.rand(n)
    logits = row.expand(n, V).contiguous().to(DEV)
    args = (torch.full((n,), 0.9, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
            torch.ones(n, device=DEV))
    got = ops().sample(logits, *args, u.to(DEV)).cpu()
    one = ops().sample(logits[:1].contiguous(), args[0][:1], args[1][:1], args[2][:1], u[:1].to(DEV)).cpu()
    assert one[0] == got[0]
    probs = torch.softmax(row.double() / 0.9, dim=0)
    top = torch.argsort(probs, descending=True)[:5]
    freq = torch.bincount(got.long(), minlength=V).double() / n
    for tkn in top.tolist():
        assert abs(freq[tkn] - probs[tkn]) < 4 * math.sqrt(probs[tkn] * (1 - probs[tkn]) / n) + 1e-3


def test_repetition_penalty():
    logits = torch.tensor([[1.0, -2.0, 4.0, 0.5], [3.0, 3.0, -1.0, 2.0]], device=DEV)
    ops().apply_penalty(logits, torch.tensor([0, 0, 1], dtype=torch.int32, device=DEV),
                        torch.tensor([1, 2, 0], dtype=torch.int32, device=DEV),
                        torch.tensor([2.0, 2.0, 1.5], device=DEV))
    assert logits.cpu().tolist() == [[1.0, -4.0, 2.0, 0.5], [2.0, 3.0, -1.0, 2.0]]


def test_repetition_penalty_from_the_table_of_seen_tokens():
    """seen_mark + penalty_seen do what apply_penalty does with host lists: every token a slot
    has seen once, rows without a slot untouched, a vocabulary that is no multiple of four."""
    o = ops()
    V, slots_n = 1003, 5
    g = torch.Generator().manual_seed(3)
    seen = torch.zeros(slots_n, 1008, dtype=torch.uint8, device=DEV)
    hist = {1: [5, 5, 1002, 17, 0], 3: [999, 1001, 4]}
    for slot, toks in hist.items():
        o.seen_mark(seen, torch.tensor(toks, dtype=torch.int32, device=DEV), None, slot)
    # marks by row: (slot, token) pairs, a slot of -1 is skipped
    o.seen_mark(seen, torch.tensor([7, 8, 9], dtype=torch.int32, device=DEV),
                torch.tensor([1, -1, 3], dtype=torch.int32, device=DEV))
    hist[1].append(7); hist[3].append(9)
    assert int(seen.sum()) == len(set(hist[1])) + len(set(hist[3]))
    logits = torch.randn(4, V, generator=g)
    want = logits.clone()
    row_slots, pens = [3, -1, 1, 1], [1.5, 2.0, 0.5, 1.3]
    for r, (sl, pen) in enumerate(zip(row_slots, pens)):
        for t in set(hist.get(sl, [])):
            want[r, t] = want[r, t] / pen if want[r, t] > 0 else want[r, t] * pen
    got = o.penalty_seen(logits.to(DEV), seen, torch.tensor(row_slots, dtype=torch.int32, device=DEV),
                         torch.tensor(pens, device=DEV)).cpu()
    assert torch.equal(got, want)


# ------------------------------------------------------------------ weight-streaming GEMM for few rows
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(64, 64), (1000, 88), (517, 192), (4608, 3584), (320, 2368)])
def test_gemm_skinny(M, N, K):
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    b = torch.randn(N)
    want = x.double() @ w.double().t()
    scale = want.abs().max().item()
    got = ops().gemm_skinny(x.to(DEV), w.to(DEV), None, torch.float32).cpu().double()
    assert (got - want).abs().max().item() <= 1e-5 * scale * math.sqrt(K) / 8 + 1e-6   # float32 accumulation
    gotb = ops().gemm_skinny(x.to(DEV), w.to(DEV), b.to(DEV), torch.bfloat16).float().cpu().double()
    assert (gotb - (want + b.double())).abs().max().item() <= 2 ** -8 * (scale + b.abs().max().item())
    if N % 2 == 0:
        act = ops().gemm_skinny(x.to(DEV), w.to(DEV), None, torch.float32, swiglu=True).cpu()
        ref = plain.swiglu(want[:, :N // 2].float(), want[:, N // 2:].float())
        assert act.shape == (M, N // 2)
        assert (act - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())


def test_gemm_skinny_rows_do_not_depend_on_the_batch():
    torch.manual_seed(5)
    x = torch.randn(16, 3584).to(torch.bfloat16).to(DEV)
    w = (torch.randn(1003, 3584) * 0.05).to(torch.bfloat16).to(DEV)
    full = ops().gemm_skinny(x, w, None, torch.float32)
    for lo, hi in [(0, 1), (3, 8), (7, 16), (15, 16)]:
        part = ops().gemm_skinny(x[lo:hi].contiguous(), w, None, torch.float32)
        assert torch.equal(part, full[lo:hi])


# ------------------------------------------------------------------ tcgen05 GEMM for many rows
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 256, 64), (300, 1000, 200), (2048, 4608, 3584),
                                   (129, 520, 1000), (640, 3584, 18944),
                                   (8192, 4096, 64),      # seven tiles a pair of blocks: both accumulators reused
                                   (4100, 2300, 136)])    # ragged in rows, columns and K with two-SM tiles
def test_gemm_tc5(M, N, K):
    torch.manual_seed(M + N)
    x = torch.randn(M, K).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16).to(DEV)
    want = (x.double() @ w.double().t())
    scale = want.abs().max().item()
    for pair in ((False, True) if M >= 256 else (False,)):      # one block a tile; two-SM tiles
        got = ops().gemm_tc5(x, w, torch.float32, check=True, pair=pair).double()
        assert got.shape == (M, N)
        assert (got - want).abs().max().item() <= 2e-5 * scale * math.sqrt(K) / 8 + 1e-6     # float32 accumulation
        gotb = ops().gemm_tc5(x, w, torch.bfloat16, check=True, pair=pair).double()
        assert (gotb - want).abs().max().item() <= 2 ** -8 * scale
        if N % 2 == 0:
            act = ops().gemm_tc5(x, w, torch.bfloat16, swiglu=True, check=True, pair=pair).float().cpu()
            ref = plain.swiglu(want[:, :N // 2].float().cpu(), want[:, N // 2:].float().cpu())
            assert act.shape == (M, N // 2)
            assert (act - ref).abs().max().item() <= 2 ** -7 * max(1.0, ref.abs().max().item())


# ------------------------------------------------------------------ tcgen05 weight-streaming GEMM, up to 64 rows
@pytest.mark.parametrize("M,N,K", [(64, 256, 128), (1, 128, 64), (9, 1000, 200), (16, 4608, 3584), (33, 3584, 18944),
                                   (64, 37888, 3584),     # one tile a block, SwiGLU over 148 tiles
                                   (48, 152064, 512),     # several tiles a block: both accumulators reused
                                   (17, 520, 1000), (8, 1536, 8960)])
def test_gemm_stream(M, N, K):
    torch.manual_seed(M + N)
    x = torch.randn(M, K).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16).to(DEV)
    want = (x.double() @ w.double().t())
    scale = want.abs().max().item()
    got = ops().gemm_stream(x, w, torch.float32, check=True).double()
    assert got.shape == (M, N)
    assert (got - want).abs().max().item() <= 2e-5 * scale * math.sqrt(K) / 8 + 1e-6     # float32 accumulation
    again = ops().gemm_stream(x, w, torch.float32, check=True).double()
    assert torch.equal(got, again)                       # the split sums are added in a fixed order
    gotb = ops().gemm_stream(x, w, torch.bfloat16, check=True).double()
    assert (gotb - want).abs().max().item() <= 2 ** -8 * scale
    if N % 2 == 0:
        act = ops().gemm_stream(x, w, torch.bfloat16, swiglu=True, check=True).float().cpu()
        ref = plain.swiglu(want[:, :N // 2].float().cpu(), want[:, N // 2:].float().cpu())
        assert act.shape == (M, N // 2)
        assert (act - ref).abs().max().item() <= 2 ** -7 * max(1.0, ref.abs().max().item())


def test_gemm_stream_rows_do_not_depend_on_the_batch():
    """A row's outputs are the same bits whether it comes alone or among 63 others."""
    torch.manual_seed(5)
    x = torch.randn(64, 3584).to(torch.bfloat16).to(DEV)
    w = (torch.randn(3584, 3584) * 0.05).to(torch.bfloat16).to(DEV)
    full = ops().gemm_stream(x, w, torch.float32, check=True)
    for lo, hi in ((0, 1), (5, 14), (20, 53)):
        part = ops().gemm_stream(x[lo:hi].contiguous(), w, torch.float32, check=True)
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("H,KV,hd,P,window,ctxs", [
    (28, 4, 128, 16, None, [2047, 300, 0, 1, 255, 256, 257, 4000]),
    (6, 3, 48, 8, 40, [0, 5, 39, 40, 41, 100, 700]),
    (4, 2, 16, 16, None, [15, 16, 17, 2300]),
    (8, 1, 64, 32, 600, [1000, 599, 600, 601, 3000]),
    (5, 5, 256, 16, None, [20, 600]),
    (4, 2, 64, 8, None, [9000, 8191]),          # more pages a block than the kernel keeps in shared memory
    (4, 1, 128, 64, None, [200, 5000, 63, 64]),  # a page is a whole key tile
    (2, 1, 64, 128, 900, [300, 129, 2000]),      # a page is two key tiles
    (3, 1, 64, 24, None, [100, 1000]),           # a page size the tensor-map boxes do not take: rows one by one
])
@pytest.mark.parametrize("splits", [8, 4, 2, 1])
def test_attention_decode_fused(H, KV, hd, P, window, ctxs, splits):
    """One launch for bias, rotary position encoding, cache write, attention and the merge of
    the key splits of decoded tokens, against the separate kernels' plain references: the
    output, and the key and value it writes into the (NaN-filled) cache."""
    from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    o = ops()
    g = torch.Generator().manual_seed(hd + len(ctxs))
    R = len(ctxs)
    pages = sum((c + 1 + P - 1) // P for c in ctxs) + 3
    m = CacheManager([KVGroupSpec((0,), KV, hd, window)], P, pages, max_requests=32, lifo=True)
    m.set_free_order(0, torch.randperm(pages, generator=g).tolist())
    kc = torch.full((pages, KV, P, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((pages, KV, P, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    theta = 10000.0
    inv_freq = plain.rope_inv_freq(hd, theta).to(DEV)
    width = (H + 2 * KV) * hd
    qkv = (torch.randn(R, width, generator=g) * 0.7).to(torch.bfloat16)
    bias = torch.randn(width, generator=g) * 0.3
    entries, want_out, new_k, new_v = [], [], [], []
    for r, c in enumerate(ctxs):
        h = m.add_request()
        assert m.reserve(h, c + 1)
        k = torch.randn(c + 1, KV, hd, generator=g).to(torch.bfloat16)
        v = torch.randn(c + 1, KV, hd, generator=g).to(torch.bfloat16)
        row = qkv[r].float() + bias
        q_new = plain.rope_rotate_half(row[:H * hd].view(1, H, hd), torch.tensor([c]), theta).to(torch.bfloat16)
        k_new = plain.rope_rotate_half(row[H * hd:(H + KV) * hd].view(1, KV, hd), torch.tensor([c]), theta).to(torch.bfloat16)
        v_new = row[(H + KV) * hd:].view(1, KV, hd).to(torch.bfloat16)
        k[c], v[c] = k_new[0], v_new[0]
        table = m.block_table(h)
        for pos in range(c):                                   # the context; the new token's slot stays NaN
            kc[table[pos // P], :, pos % P] = k[pos].to(DEV)
            vc[table[pos // P], :, pos % P] = v[pos].to(DEV)
        m.commit(h, c)
        qfull = torch.zeros(c + 1, H, hd)
        qfull[c] = q_new[0].float()
        want_out.append(plain.causal_attention(qfull, k.float(), v.float(), hd ** -0.5, window)[c])
        new_k.append((table[c // P], c % P, k_new[0]))
        new_v.append((table[c // P], c % P, v_new[0]))
        entries.append(StepEntry(h, [0]))
    G = H // KV
    _, tile_rows, _ = o.attention_kernel_config(hd, torch.bfloat16, "mma")
    ctx = StepContext(m, entries, torch.device(DEV), [(0, G, tile_rows, window)])
    meta = ctx.attention_work(0, G, tile_rows, window, H, hd)
    assert meta.decode_rows == R
    out = torch.full((R, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.attention_decode_fused(qkv.to(DEV), bias.to(DEV), kc, vc, out, meta, ctx.positions, ctx.group(0).slots,
                             inv_freq, R, H, KV, hd, hd ** -0.5, window, P, splits=splits)
    got = out.float().cpu().view(R, H, hd)
    want = torch.stack(want_out)
    assert o.attention_mma_wait_flag(hd) == 0      # no bounded wait for a key tile ran out
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= 2 ** -6 * max(1.0, want.abs().max().item())
    for (page, off, kn), (_, _, vn) in zip(new_k, new_v):
        assert (kc[page, :, off].float().cpu() - kn.float()).abs().max().item() <= 2 ** -6 * max(1.0, kn.float().abs().max().item())
        assert torch.equal(vc[page, :, off].cpu(), vn)


@pytest.mark.parametrize("window", [None, 700])
def test_attention_decode_fused_one_key_stands_out(window):
    """One key gets all the weight (rotation switched off by zero frequencies, so that the
    score is the plain dot product): at the first key, on both sides of the kernel's own split
    boundaries (2,101 keys in 8 parts of 320; 700 in parts of 128 with the window), in the last
    page, at the new token itself, and - with a window - at the window's first key; just outside
    the window it must not be seen."""
    from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    o = ops()
    H, KV, hd, P, ctx_len = 8, 2, 64, 16, 2100
    lo = 0 if window is None else ctx_len - window + 1           # first visible key of the new token
    part = 320 if window is None else 128                         # keys per block: ceil(span / 512) * 64
    targets = [lo, lo + part - 1, lo + part, lo + 4 * part - 1, lo + 4 * part, 2099, ctx_len]   # ctx_len: its own key
    if window is not None:
        targets = [t for t in targets if t >= lo] + [lo - 1]       # the last one is outside the window
    R = len(targets)
    g = torch.Generator().manual_seed(5)
    pages = R * ((ctx_len + 1 + P - 1) // P) + 2
    m = CacheManager([KVGroupSpec((0,), KV, hd, window)], P, pages, max_requests=R)
    kc = torch.full((pages, KV, P, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((pages, KV, P, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    width = (H + 2 * KV) * hd
    qkv = torch.zeros(R, width)
    qkv[:, 0:H * hd:hd] = 40.0                                     # every query head: 40 e0
    entries, values = [], []
    for r, j in enumerate(targets):
        h = m.add_request()
        assert m.reserve(h, ctx_len + 1)
        k = torch.randn(ctx_len + 1, KV, hd, generator=g) * 0.05
        v = torch.randn(ctx_len + 1, KV, hd, generator=g)
        k[:, :, 0] = 0
        if j < ctx_len:
            k[j, :, 0] = 8.0
        else:
            qkv[r, H * hd:(H + KV) * hd:hd] = 8.0                  # the new token's own key stands out
        new_v = torch.randn(KV, hd, generator=g)
        qkv[r, (H + KV) * hd:] = new_v.reshape(-1)
        v[ctx_len] = new_v
        table = m.block_table(h)
        for pos in range(ctx_len):
            kc[table[pos // P], :, pos % P] = k[pos].to(torch.bfloat16).to(DEV)
            vc[table[pos // P], :, pos % P] = v[pos].to(torch.bfloat16).to(DEV)
        m.commit(h, ctx_len)
        values.append(v[j].to(torch.bfloat16).float())
        entries.append(StepEntry(h, [0]))
    G = H // KV
    _, tile_rows, _ = o.attention_kernel_config(hd, torch.bfloat16, "mma")
    ctx = StepContext(m, entries, torch.device(DEV), [(0, G, tile_rows, window)])
    meta = ctx.attention_work(0, G, tile_rows, window, H, hd)
    out = torch.full((R, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    inv_freq = torch.zeros(hd // 2, device=DEV)
    o.attention_decode_fused(qkv.to(torch.bfloat16).to(DEV), None, kc, vc, out, meta, ctx.positions,
                             ctx.group(0).slots, inv_freq, R, H, KV, hd, hd ** -0.5, window, P, splits=8)
    got = out.float().cpu().view(R, H, hd)
    assert torch.isfinite(got).all()
    for r, j in enumerate(targets):
        seen = window is None or j >= lo
        for head in range(H):
            close = torch.allclose(got[r, head], values[r][head // G], atol=3e-2)
            assert close == seen, (r, j, head, seen)

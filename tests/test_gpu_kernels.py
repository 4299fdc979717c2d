"""Each kernel alone against a plain PyTorch float32 (or float64) reference of the same
operation, at sizes other than the engine's tiny models: widths and vocabularies that are
no power of two, head sizes in steps of 16, several group sizes, scattered cache pages."""
from __future__ import annotations

import math

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
PAGE = 64


def _tol(dtype):
    return {"float32": 1e-5, "bfloat16": 1.6e-2}[dtype]


def _close(got, ref, dtype, what, scale=None):
    got, ref = got.float().cpu(), ref.float().cpu()
    scale = float(ref.abs().max()) if scale is None else scale
    err = float((got - ref).abs().max())
    assert err <= _tol(dtype) * scale + 1e-7, f"{what}: max abs error {err:.3e}, scale {scale:.3e}"


@pytest.fixture(scope="module")
def ops():
    from kuiperllama_b200.csrc import ops
    return ops


# ----------------------------------------------------------------------------- embedding

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_gathers_rows_and_flags_bad_ids(ops, dtype):
    torch.manual_seed(0)
    table = torch.randn(1003, 96, device=DEV).to(DT[dtype])
    ids = torch.tensor([5, 1002, 0, 77, 5], dtype=torch.int32, device=DEV)
    out = torch.full((5, 96), 7.0, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embedding(ids, table, out, flag)
    assert torch.equal(out, plain_llama.embedding(table.float().cpu(), ids.tolist()).to(DEV)) and int(flag) == 0
    bad = torch.tensor([3, 1003, -1], dtype=torch.int32, device=DEV)
    ops.embedding(bad, table, out, flag)
    assert int(flag) == 1 and torch.equal(out[0], table[3].float()) and float(out[1:3].abs().sum()) == 0.0


# ----------------------------------------------------------------------------- norm

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [100, 4096, 8200])
def test_add_rmsnorm(ops, dtype, hidden):
    torch.manual_seed(1)
    T, eps = 37, 3e-6
    resid = torch.randn(T, hidden, device=DEV) * 3
    delta = (torch.randn(T, hidden, device=DEV)).to(DT[dtype])
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    out = torch.empty(T, hidden, device=DEV, dtype=DT[dtype])
    r0 = resid.clone()
    ops.add_rmsnorm(resid, None, w, out, eps)                                   # no delta: the stream is untouched
    assert torch.equal(resid, r0)
    _close(out, plain_llama.rmsnorm(r0.cpu(), w.cpu(), eps), dtype, "rmsnorm")
    ops.add_rmsnorm(resid, delta, w, out, eps)                                  # with delta: written back in float32
    x = r0 + delta.float()
    assert torch.equal(resid, x), "the residual sum is not the float32 sum"
    _close(out, plain_llama.rmsnorm(x.cpu(), w.cpu(), eps), dtype, "add+rmsnorm")
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32, device=DEV)
    out2 = torch.empty(4, hidden, device=DEV, dtype=DT[dtype])
    before = resid.clone()
    ops.add_rmsnorm(resid, delta, w, out2, eps, rows)                           # a few rows, nothing written back
    assert torch.equal(resid, before)
    x2 = (before + delta.float())[rows.long()]
    _close(out2, plain_llama.rmsnorm(x2.cpu(), w.cpu(), eps), dtype, "gathered rows")
    # a delta given as float32 partial sums [S, rows, hidden], added in ascending order
    parts = torch.randn(3, T, hidden, device=DEV)
    before = resid.clone()
    ops.add_rmsnorm(resid, parts, w, out, eps)
    x3 = ((before + parts[0]) + parts[1]) + parts[2]
    assert torch.equal(resid, x3), "partial sums are not added in ascending order in float32"
    _close(out, plain_llama.rmsnorm(x3.cpu(), w.cpu(), eps), dtype, "partial sums + rmsnorm")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(ops, dtype):
    torch.manual_seed(2)
    T, I = 19, 173
    gu = (torch.randn(T, 2 * I, device=DEV) * 4).to(DT[dtype])
    out = torch.empty(T, I, device=DEV, dtype=DT[dtype])
    ops.swiglu(gu, out)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    _close(out, g * (1 / (1 + torch.exp(-g))) * u, dtype, "swiglu")


# ----------------------------------------------------------------------------- matrix product

@pytest.mark.parametrize("dtype,out_dtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("bfloat16", "float32")])
@pytest.mark.parametrize("M,N,K", [(1, 1003, 172), (3, 65, 64), (70, 130, 333), (129, 64, 16), (64, 256, 4100)])
def test_gemm_simt(ops, dtype, out_dtype, M, N, K):
    torch.manual_seed(3)
    a = torch.randn(M, K, device=DEV).to(DT[dtype])
    w = torch.randn(N, K, device=DEV).to(DT[dtype])
    out = torch.empty(M, N, device=DEV, dtype=DT[out_dtype])
    ops.gemm_simt(a, w, out)
    ref = (a.double().cpu() @ w.double().cpu().T)
    # A true 32-bit product.  A float32 sum of K terms taken one after the other carries a
    # rounding error of about 2^-24 * sqrt(K) relative to the partial sums; a reduced-precision
    # matrix mode (tf32: 2^-11 per product) would be off by about 2^-11 * sqrt(K) of one term,
    # more than ten times the bound below.
    tol = {"float32": 2.0 * 2.0 ** -24 * math.sqrt(K), "bfloat16": 8e-3}[out_dtype]
    err = float((out.double().cpu() - ref).abs().max())
    assert err <= tol * float(ref.abs().max()), f"gemm {M}x{N}x{K} {dtype}->{out_dtype}: error {err:.3e}"


def test_gemm_rows_do_not_depend_on_the_batch(ops):
    torch.manual_seed(4)
    a = torch.randn(70, 333, device=DEV)
    w = torch.randn(130, 333, device=DEV)
    full = torch.empty(70, 130, device=DEV)
    ops.gemm_simt(a, w, full)
    one = torch.empty(1, 130, device=DEV)
    ops.gemm_simt(a[41:42].contiguous(), w, one)
    assert torch.equal(one[0], full[41])


# ----------------------------------------------------------------------------- rope + cache write, attention

class Paged:
    """A scattered paged cache for tests: pages are dealt to slots in shuffled order."""

    def __init__(self, n_slots, max_len, KV, hd, dtype, seed=0):
        self.blocks = (max_len + PAGE - 1) // PAGE
        n_pages = n_slots * self.blocks + 3
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(n_pages, generator=g)[: n_slots * self.blocks]
        self.table = perm.view(n_slots, self.blocks).to(torch.int32).to(DEV)
        # stale contents everywhere: large values that would show if they were read
        self.k = (torch.randn(n_pages, KV, PAGE, hd, generator=g) * 50).to(dtype).to(DEV)
        self.v = (torch.randn(n_pages, KV, PAGE, hd, generator=g) * 50).to(dtype).to(DEV)

    def rows(self, which, slot, length):
        """[length, KV, hd] of a slot, gathered on the host."""
        t = self.table[slot].tolist()
        src = (self.k if which == "k" else self.v).float().cpu()
        return torch.stack([src[t[p // PAGE], :, p % PAGE, :] for p in range(length)], dim=0)


def _ref_rope(x, positions, inv_freq, rot):
    """x [T, heads, hd]: rotate the first `rot` elements of every head, half-split pairs."""
    if rot == 0:
        return x.clone()
    out = x.clone()
    out[..., :rot] = plain_llama.rope_rotate(x[..., :rot], positions, inv_freq)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,rot", [(4, 4, 16, 16), (6, 2, 32, 32), (8, 2, 128, 128), (5, 1, 48, 24), (3, 3, 80, 0)])
def test_rope_kv_write(ops, dtype, H, KV, hd, rot):
    torch.manual_seed(5)
    dt = DT[dtype]
    lens = [70, 1, 130]                                           # tokens of three sequences, appended at offsets
    starts = [60, 0, 3]
    cache = Paged(4, 256, KV, hd, dt, seed=1)
    slots = [2, 0, 3]
    T = sum(lens)
    qkv = torch.randn(T, (H + 2 * KV) * hd, device=DEV).to(dt)
    pos = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=DEV)
    tslot = torch.tensor([sl for sl, n in zip(slots, lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    # padding rows: slot -1 must write nothing and leave q alone
    qkv = torch.cat([qkv, torch.ones(2, qkv.shape[1], device=DEV, dtype=dt)])
    pos = torch.cat([pos, torch.zeros(2, dtype=torch.int32, device=DEV)])
    tslot = torch.cat([tslot, torch.full((2,), -1, dtype=torch.int32, device=DEV)])
    inv = plain_llama.rope_inverse_frequencies(rot, 500000.0, None).to(DEV) if rot else None
    before_k, before_v = cache.k.clone(), cache.v.clone()
    x = qkv.clone()
    ops.rope_kv_write(x, inv, rot, pos, tslot, cache.table, cache.k, cache.v, H, KV, hd)
    src = qkv[:T].float().cpu().view(T, H + 2 * KV, hd)
    p = pos[:T].cpu()
    invc = inv.cpu() if rot else None
    q_ref = _ref_rope(src[:, :H], p, invc, rot)
    k_ref = _ref_rope(src[:, H:H + KV], p, invc, rot)
    v_ref = src[:, H + KV:]
    _close(x[:T].view(T, H + 2 * KV, hd)[:, :H], q_ref, dtype, "rotated q", scale=float(src.abs().max()))
    assert torch.equal(x[T:], qkv[T:]), "a padding row was touched"
    o = 0
    written = torch.zeros_like(cache.k, dtype=torch.bool)
    for sl, st, n in zip(slots, starts, lens):
        rows_k, rows_v = cache.rows("k", sl, st + n), cache.rows("v", sl, st + n)
        _close(rows_k[st:], k_ref[o:o + n], dtype, f"keys of slot {sl}", scale=float(src.abs().max()))
        assert torch.equal(rows_v[st:], v_ref[o:o + n].to(dt).float()), "values must be stored as they are"
        for i in range(st, st + n):
            written[cache.table[sl, i // PAGE], :, i % PAGE, :] = True
        o += n
    assert torch.equal(cache.k[~written], before_k[~written]) and torch.equal(cache.v[~written], before_v[~written]), \
        "something outside the new tokens' rows was written"
    # the same projections given as three float32 pieces: same queries and cache rows
    cache2 = Paged(4, 256, KV, hd, dt, seed=1)
    full = qkv.float()
    pieces = torch.randn(3, *full.shape, device=DEV)
    pieces[2] = full - (pieces[0] + pieces[1])
    exact = ((pieces[0] + pieces[1]) + pieces[2])
    y = torch.zeros_like(qkv)
    ops.rope_kv_write(y, inv, rot, pos, tslot, cache2.table, cache2.k, cache2.v, H, KV, hd, partials=pieces)
    src2 = exact[:T].cpu().view(T, H + 2 * KV, hd)
    _close(y[:T].view(T, H + 2 * KV, hd)[:, :H], _ref_rope(src2[:, :H], p, invc, rot), dtype, "rotated q from pieces",
           scale=float(src.abs().max()))
    o = 0
    for sl, st, n in zip(slots, starts, lens):
        _close(cache2.rows("k", sl, st + n)[st:], _ref_rope(src2[:, H:H + KV], p, invc, rot)[o:o + n], dtype,
               f"keys of slot {sl} from pieces", scale=float(src.abs().max()))
        _close(cache2.rows("v", sl, st + n)[st:], src2[:, H + KV:][o:o + n], dtype, f"values of slot {sl} from pieces",
               scale=float(src.abs().max()))
        o += n


def _fill_cache(cache, slot, k, v):
    """k, v: [len, KV, hd] float tensors -> the slot's pages."""
    t = cache.table[slot].tolist()
    for p in range(k.shape[0]):
        cache.k[t[p // PAGE], :, p % PAGE, :] = k[p].to(cache.k.dtype).to(DEV)
        cache.v[t[p // PAGE], :, p % PAGE, :] = v[p].to(cache.v.dtype).to(DEV)


def _ref_attention(q, k, v, pos, scale, window):
    """q [H, hd] of one token at position pos; k, v [len, KV, hd]."""
    H, hd = q.shape
    KV = k.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    out = torch.empty(H, hd, dtype=torch.float64)
    for h in range(H):
        g = h // (H // KV)
        s = (k[lo:pos + 1, g].double() @ q[h].double()) * scale
        p = torch.softmax(s, dim=0)
        out[h] = p @ v[lo:pos + 1, g].double()
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,window", [(4, 4, 16, 0), (6, 2, 32, 0), (8, 2, 128, 0), (3, 1, 48, 0), (4, 2, 80, 0),
                                            (2, 1, 256, 0), (4, 2, 64, 37), (12, 4, 96, 0)])
def test_attention_simt(ops, dtype, H, KV, hd, window):
    torch.manual_seed(6)
    dt = DT[dtype]
    lens = [200, 1, 65, 129]
    cache = Paged(5, 256, KV, hd, dt, seed=2)
    slots = [4, 1, 0, 2]
    ks = [torch.randn(n, KV, hd) for n in lens]
    vs = [torch.randn(n, KV, hd) for n in lens]
    for sl, k, v in zip(slots, ks, vs):
        _fill_cache(cache, sl, k, v)
    # query tokens: several positions of every sequence, in one packed batch, plus a padding row
    picks = [(0, 199), (0, 0), (0, 63), (0, 64), (1, 0), (2, 64), (2, 31), (3, 128), (3, 127), (0, 100)]
    T = len(picks)
    scale = 1.0 / math.sqrt(hd)
    stride = H * hd + 24                                            # q rows inside a wider buffer
    qbuf = torch.randn(T + 1, stride, device=DEV).to(dt)
    pos = torch.tensor([p for _, p in picks] + [0], dtype=torch.int32, device=DEV)
    tslot = torch.tensor([slots[i] for i, _ in picks] + [-1], dtype=torch.int32, device=DEV)
    out = torch.full((T + 1, H * hd), 3.0, device=DEV, dtype=dt)
    ops.attention_simt(qbuf, stride, out, cache.k, cache.v, cache.table, pos, tslot, T + 1, H, KV, hd, scale, window)
    assert float((out[T].float() - 3.0).abs().max()) == 0.0, "a padding row was written"
    for t, (i, p) in enumerate(picks):
        q = qbuf[t, :H * hd].float().cpu().view(H, hd)
        kk = ks[i].to(dt).float()
        vv = vs[i].to(dt).float()
        ref = _ref_attention(q, kk, vv, p, scale, window)
        _close(out[t].view(H, hd), ref, dtype, f"attention token {t} (seq {i}, pos {p})", scale=float(vv.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(ops, dtype):
    """One key far back is made to dominate the softmax; the output must be its value.  A
    kernel that skips a chunk, misreads a page or stops early returns something else."""
    torch.manual_seed(7)
    dt = DT[dtype]
    H, KV, hd, n = 4, 2, 64, 900
    cache = Paged(2, 1024, KV, hd, dt, seed=3)
    k = torch.randn(n, KV, hd) * 0.1
    v = torch.randn(n, KV, hd)
    q = torch.randn(H, hd) * 0.1
    for far in (0, 63, 64, 517, 899):
        kk = k.clone()
        kk[far, :, :] = 0
        kk[far, :, 5] = 40.0
        qq = q.clone()
        qq[:, 5] = 40.0                                             # score 1600 / 8 = 200 at the far key
        _fill_cache(cache, 1, kk, v)
        qbuf = qq.view(1, H * hd).to(dt).to(DEV)
        out = torch.empty(1, H * hd, device=DEV, dtype=dt)
        pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        tslot = torch.tensor([1], dtype=torch.int32, device=DEV)
        ops.attention_simt(qbuf, H * hd, out, cache.k, cache.v, cache.table, pos, tslot, 1, H, KV, hd, 1 / 8.0, 0)
        want = v[far].to(dt).float().repeat_interleave(H // KV, dim=0)
        _close(out.view(H, hd), want, dtype, f"far key at {far}")


# ----------------------------------------------------------------------------- sampling

def test_argmax_rows_lowest_index_among_equals(ops):
    torch.manual_seed(8)
    logits = torch.randn(7, 128256, device=DEV)
    logits[2, 99999] = 50.0
    logits[3, [5, 70000, 128255]] = 60.0                           # equal maxima: the lowest index wins
    logits[4, 128255] = 70.0
    out = torch.empty(7, dtype=torch.int32, device=DEV)
    ops.argmax_rows(logits, out)
    want = [plain_llama.argmax_token(r) for r in logits.cpu()]
    assert out.tolist() == want and want[2] == 99999 and want[3] == 5 and want[4] == 128255
    wide = torch.randn(3, 1003 + 21, device=DEV)[:, :1003]          # rows with a stride
    out3 = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax_rows(wide, out3)
    assert out3.tolist() == wide.argmax(dim=1).tolist()


@pytest.mark.parametrize("vocab,temperature,top_k", [(1003, 0.8, 0), (128256, 1.0, 0), (384, 0.5, 5), (5000, 1.3, 50),
                                                     (777, 2.0, 1)])
def test_sample_rows_is_the_inverse_cdf_of_the_counter_draw(ops, vocab, temperature, top_k):
    torch.manual_seed(9)
    rows, seed = 24, 1234
    logits = torch.randn(rows, vocab, device=DEV) * 3
    req = torch.arange(100, 100 + rows, dtype=torch.int32, device=DEV)
    steps = torch.arange(rows, dtype=torch.int32, device=DEV) % 5
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits, temperature, top_k, seed, req, steps, out)
    again = torch.empty_like(out)
    ops.sample_rows(logits.clone(), temperature, top_k, seed, req, steps, again)
    assert torch.equal(out, again)
    for r in range(rows):
        p = plain_llama.temperature_probabilities(logits[r].cpu(), temperature, top_k or None)
        u = plain_llama.uniform_from_counter(seed, int(req[r]), int(steps[r]))
        c = torch.cumsum(p, 0)
        got = int(out[r])
        # the chosen token's interval of the cumulative distribution holds u (up to float rounding)
        lo = float(c[got - 1]) if got > 0 else 0.0
        assert float(p[got]) > 0 and lo - 1e-5 <= u <= float(c[got]) + 1e-5, (r, got, u, lo, float(c[got]))
        if top_k == 1:
            assert got == plain_llama.argmax_token(logits[r].cpu())
    # a row's draw depends on its request id and step, not on its place in the batch
    sub = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits[7:8], temperature, top_k, seed, req[7:8].contiguous(), steps[7:8].contiguous(), sub)
    assert int(sub) == int(out[7])


# ----------------------------------------------------------------------------- tensor-core products

@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
# Shapes with an even number of 128-token tiles (or 1,024 tokens and more) run on pairs of CTAs with tiles
# of 256 x 256, the others on single CTAs with tiles of 128 x 256; ragged edges in both directions for both.
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (65, 72, 136), (300, 1000, 520), (2048, 512, 4096), (129, 257, 72),
                                   (1000, 130, 1024), (2048, 4096, 512), (2000, 5000, 2056), (700, 4096, 1024), (1100, 300, 264),
                                   (640, 4096, 8192)])
def test_gemm_tcgen05(ops, out_dtype, M, N, K):
    torch.manual_seed(10)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    ref = a.double().cpu() @ w.double().cpu().T
    tol = {"float32": 2.0 * 2.0 ** -24 * math.sqrt(K), "bfloat16": 8e-3}[out_dtype]
    outs = []
    for _ in range(2):
        out = torch.full((M, N), 7.0, device=DEV, dtype=DT[out_dtype])
        ops.gemm_tcgen05(a, w, out)
        ops.check_status(out.device)
        err = float((out.double().cpu() - ref).abs().max())
        assert err <= tol * float(ref.abs().max()), f"tcgen05 gemm {M}x{N}x{K} -> {out_dtype}: error {err:.3e}"
        outs.append(out)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("M,N,K,splits", [(1, 128, 64, 1), (8, 4096, 4096, None), (16, 1000, 520, 3), (17, 130, 1024, 4),
                                          (33, 257, 72, 2), (64, 6144, 4096, None), (5, 1003, 14336, None), (3, 200, 64, 1),
                                          # more than 64 tokens: several tiles of 64 tokens per weight tile
                                          (65, 300, 264, 1), (96, 4096, 4096, None), (128, 1000, 520, 3), (200, 130, 1024, 4),
                                          (256, 6144, 2048, None), (129, 257, 72, 1), (300, 1000, 520, 2), (512, 4096, 4096, None)])
def test_gemm_skinny(ops, out_dtype, M, N, K, splits):
    torch.manual_seed(11)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    out = torch.full((M, N), 7.0, device=DEV, dtype=DT[out_dtype])
    ops.gemm_skinny(a, w, out, splits)
    ops.check_status(out.device)
    ref = a.double().cpu() @ w.double().cpu().T
    tol = {"float32": 2.0 * 2.0 ** -24 * math.sqrt(K), "bfloat16": 8e-3}[out_dtype]
    err = float((out.double().cpu() - ref).abs().max())
    assert err <= tol * float(ref.abs().max()), f"skinny gemm {M}x{N}x{K} -> {out_dtype}: error {err:.3e}"


def test_matmul_picks_a_kernel_for_every_shape(ops):
    """Rows that are not 16-byte aligned (K = 172) go to the plain kernel, never to a wrong result."""
    torch.manual_seed(12)
    for M, N, K in [(5, 64, 172), (100, 64, 172), (5, 172, 64), (100, 172, 64)]:
        a = torch.randn(M, K, device=DEV).bfloat16()
        w = torch.randn(N, K, device=DEV).bfloat16()
        out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        ops.matmul(a, w, out)
        ref = a.double().cpu() @ w.double().cpu().T
        assert float((out.double().cpu() - ref).abs().max()) <= 8e-3 * float(ref.abs().max())
    ops.check_status(torch.device(DEV))


# ----------------------------------------------------------------------------- split-KV decode attention

@pytest.mark.parametrize("H,KV,hd,window,splits", [(4, 4, 16, 0, 1), (6, 2, 32, 0, 3), (8, 2, 128, 0, None), (32, 8, 128, 0, 5),
                                                   (3, 1, 64, 0, 2), (16, 2, 64, 0, 4), (2, 1, 256, 0, 7), (4, 2, 64, 37, 3),
                                                   (8, 8, 128, 100, 32), (5, 5, 32, 0, 32)])
def test_attention_decode(ops, H, KV, hd, window, splits):
    torch.manual_seed(13)
    dt = torch.bfloat16
    lens = [200, 1, 65, 129, 64, 250]
    cache = Paged(7, 256, KV, hd, dt, seed=4)
    slots = [4, 1, 0, 2, 6, 5]
    ks = [torch.randn(n, KV, hd) for n in lens]
    vs = [torch.randn(n, KV, hd) for n in lens]
    for sl, k, v in zip(slots, ks, vs):
        _fill_cache(cache, sl, k, v)
    rows = len(lens) + 1                                            # the last token of every sequence, one padding row
    stride = H * hd + 2 * KV * hd
    qbuf = torch.randn(rows, stride, device=DEV).to(dt)
    pos = torch.tensor([n - 1 for n in lens] + [0], dtype=torch.int32, device=DEV)
    tslot = torch.tensor(slots + [-1], dtype=torch.int32, device=DEV)
    out = torch.full((rows, H * hd), 3.0, device=DEV, dtype=dt)
    ops.attention_decode(qbuf, stride, out, cache.k, cache.v, cache.table, pos, tslot, rows, H, KV, hd, 1 / math.sqrt(hd),
                         window, splits)
    assert float((out[-1].float() - 3.0).abs().max()) == 0.0, "a padding row was written"
    for t, n in enumerate(lens):
        q = qbuf[t, :H * hd].float().cpu().view(H, hd)
        ref = _ref_attention(q, ks[t].to(dt).float(), vs[t].to(dt).float(), n - 1, 1 / math.sqrt(hd), window)
        _close(out[t].view(H, hd), ref, "bfloat16", f"decode attention row {t} (len {n})", scale=float(vs[t].abs().max()))


@pytest.mark.parametrize("splits", [1, 4, 32])
def test_attention_decode_finds_one_far_key_among_thousands(ops, splits):
    torch.manual_seed(14)
    dt = torch.bfloat16
    H, KV, hd, n = 8, 2, 128, 3000
    cache = Paged(2, 3072, KV, hd, dt, seed=5)
    k = torch.randn(n, KV, hd) * 0.1
    v = torch.randn(n, KV, hd)
    q = torch.randn(H, hd) * 0.1
    q[:, 9] = 40.0
    for far in (0, 63, 64, 1999, 2999):
        kk = k.clone()
        kk[far] = 0
        kk[far, :, 9] = 40.0
        _fill_cache(cache, 1, kk, v)
        qbuf = q.view(1, H * hd).to(dt).to(DEV)
        out = torch.empty(1, H * hd, device=DEV, dtype=dt)
        pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        tslot = torch.tensor([1], dtype=torch.int32, device=DEV)
        ops.attention_decode(qbuf, H * hd, out, cache.k, cache.v, cache.table, pos, tslot, 1, H, KV, hd, 1 / math.sqrt(hd), 0, splits)
        want = v[far].to(dt).float().repeat_interleave(H // KV, dim=0)
        _close(out.view(H, hd), want, "bfloat16", f"far key at {far}, {splits} splits")


# ----------------------------------------------------------------------------- tensor-core attention

def _ragged_problem(H, KV, hd, seqs, seed):
    """seqs: [(start, new)] per sequence.  Fills the cache with start + new keys per sequence."""
    torch.manual_seed(seed)
    dt = torch.bfloat16
    n = len(seqs)
    cache = Paged(n + 1, max(s + t for s, t in seqs) + 1, KV, hd, dt, seed=seed)
    slots = list(range(n, 0, -1))
    ks = [torch.randn(s + t, KV, hd) for s, t in seqs]
    vs = [torch.randn(s + t, KV, hd) for s, t in seqs]
    for sl, k, v in zip(slots, ks, vs):
        _fill_cache(cache, sl, k, v)
    rows = sum(t for _, t in seqs)
    stride = (H + 2 * KV) * hd
    qbuf = torch.randn(rows + 2, stride, device=DEV).to(dt)           # two padding rows at the end
    cu = [0]
    for _, t in seqs:
        cu.append(cu[-1] + t)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return cache, slots, ks, vs, qbuf, stride, i32(cu), i32(slots), i32([s for s, _ in seqs]), i32([t for _, t in seqs]), rows


@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 128, 0), (4, 4, 64, 0), (6, 2, 64, 0), (32, 8, 128, 0), (8, 1, 128, 0),
                                            (4, 2, 128, 50), (16, 1, 64, 0)])
def test_attention_mma_prefill(ops, H, KV, hd, window):
    seqs = [(0, 150), (0, 1), (60, 70), (3, 64), (0, 65), (100, 5)]
    cache, slots, ks, vs, qbuf, stride, cu, sl, st, nw, rows = _ragged_problem(H, KV, hd, seqs, seed=15)
    out = torch.full((rows + 2, H * hd), 3.0, device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    ops.attention_mma(qbuf, stride, out, cache.k, cache.v, cache.table, cu, sl, st, nw, len(seqs), max(t for _, t in seqs),
                      rows, H, KV, hd, scale, window, 1, False)
    assert float((out[rows:].float() - 3.0).abs().max()) == 0.0, "a padding row was written"
    r = 0
    for i, (s0, t) in enumerate(seqs):
        kk, vv = ks[i].bfloat16().float(), vs[i].bfloat16().float()
        for j in range(t):
            qv = qbuf[r, :H * hd].float().cpu().view(H, hd)
            ref = _ref_attention(qv, kk, vv, s0 + j, scale, window)
            _close(out[r].view(H, hd), ref, "bfloat16", f"mma prefill seq {i} token {j}", scale=float(vv.abs().max()))
            r += 1


# the cases with 7 * KV * splits > 444 take the light CTAs (two warps, half pages) of the head size 128
@pytest.mark.parametrize("H,KV,hd,window,splits", [(8, 2, 128, 0, 1), (32, 8, 128, 0, 5), (4, 4, 64, 0, 3), (6, 2, 64, 0, 16),
                                                   (8, 8, 128, 100, 2), (16, 1, 128, 0, 4), (32, 8, 128, 0, 9), (8, 8, 128, 100, 8),
                                                   (64, 64, 128, 0, 2), (24, 8, 128, 33, 16),
                                                   # 592 < 7 * KV * splits <= 888: light CTAs of two stages, six per SM
                                                   (32, 8, 128, 0, 12), (8, 8, 128, 100, 11)])
def test_attention_mma_decode(ops, H, KV, hd, window, splits):
    seqs = [(199, 1), (0, 1), (64, 1), (128, 1), (63, 1), (249, 1), (1000, 1)]
    cache, slots, ks, vs, qbuf, stride, cu, sl, st, nw, rows = _ragged_problem(H, KV, hd, seqs, seed=16)
    out = torch.full((rows + 2, H * hd), 3.0, device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    ops.attention_mma(qbuf, stride, out, cache.k, cache.v, cache.table, cu, sl, st, nw, len(seqs), 1, rows, H, KV, hd, scale,
                      window, splits, True)
    for i, (s0, _) in enumerate(seqs):
        qv = qbuf[i, :H * hd].float().cpu().view(H, hd)
        ref = _ref_attention(qv, ks[i].bfloat16().float(), vs[i].bfloat16().float(), s0, scale, window)
        _close(out[i].view(H, hd), ref, "bfloat16", f"mma decode seq {i} (len {s0 + 1})", scale=float(vs[i].abs().max()))


@pytest.mark.parametrize("few_rows,splits,KV", [(False, 1, 2), (True, 1, 2), (True, 7, 2), (True, 29, 16), (True, 40, 16)])
def test_attention_mma_finds_one_far_key_among_thousands(ops, few_rows, splits, KV):
    """With 16 kv heads and 29 or 40 pieces the decode layout's light CTAs run (half pages; four or six
    per SM): the far keys also sit at the ends of half pages."""
    torch.manual_seed(17)
    dt = torch.bfloat16
    H, hd, n = max(8, KV), 128, 3000
    for far in (0, 31, 32, 63, 64, 1999, 2975, 2976, 2999):
        cache = Paged(2, 3072, KV, hd, dt, seed=6)
        k = torch.randn(n, KV, hd) * 0.1
        v = torch.randn(n, KV, hd)
        k[far] = 0
        k[far, :, 9] = 40.0
        _fill_cache(cache, 1, k, v)
        new = 1 if few_rows else 20                                  # the last `new` tokens are the queries
        q = torch.randn(new, H, hd) * 0.1
        q[:, :, 9] = 40.0
        qbuf = q.view(new, H * hd).to(dt).to(DEV)
        out = torch.empty(new, H * hd, device=DEV, dtype=dt)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        ops.attention_mma(qbuf, H * hd, out, cache.k, cache.v, cache.table, i32([0, new]), i32([1]), i32([n - new]), i32([new]),
                          1, new, new, H, KV, hd, 1 / math.sqrt(hd), 0, splits, few_rows)
        want = v[far].to(dt).float().repeat_interleave(H // KV, dim=0)
        for j in range(new):
            if far <= n - new + j:
                _close(out[j].view(H, hd), want, "bfloat16", f"far key at {far}, query {j}")


@pytest.mark.parametrize("kernel", ["simt_f32", "simt_bf16", "decode_split", "mma_prefill", "mma_decode", "fused_decode"])
@pytest.mark.parametrize("window,n", [(100, 300), (64, 129), (65, 200), (1, 70)])
def test_the_windows_edge_is_exact(ops, kernel, window, n):
    """One key is made to dominate the softmax: first the key just outside the last query's
    window (position p - window), which must not be seen at all, then the window's first key
    (p - window + 1), whose value the output must then be.  Random scores would hide an edge
    that is off by one inside the tolerance."""
    from types import SimpleNamespace
    torch.manual_seed(31)
    H, KV, hd = 4, 2, 64
    dt = torch.float32 if kernel == "simt_f32" else torch.bfloat16
    name = "float32" if kernel == "simt_f32" else "bfloat16"
    scale = 1 / math.sqrt(hd)
    p_last = n - 1
    new = 20 if kernel == "mma_prefill" else 1                  # query tokens: the last `new` positions
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    for edge in (p_last - window, p_last - window + 1):
        if edge < 0:
            continue
        k = torch.randn(n, KV, hd) * 0.1
        v = torch.randn(n, KV, hd)
        k[edge] = 0
        k[edge, :, 9] = 40.0
        q = torch.randn(new, H, hd) * 0.1
        q[:, :, 9] = 40.0                                       # score 1600 / 8 = 200 at the edge key
        cache = Paged(2, 320, KV, hd, dt, seed=8)
        out = torch.empty(new, H * hd, device=DEV, dtype=dt)
        if kernel == "fused_decode":
            # the kernel writes the last token's key and value itself: give them as the projection's k and v
            _fill_cache(cache, 1, k[:-1], v[:-1])
            inv = torch.zeros(hd // 2, device=DEV)               # no rotation: angles are all zero
            qkv = torch.cat([q[0].reshape(-1), k[-1].reshape(-1), v[-1].reshape(-1)])[None].to(dt).to(DEV)
            step = SimpleNamespace(n_seqs=1, n_tokens=1, is_decode=True, cu_tokens=i32([0, 1]), seq_slots=i32([1]),
                                   seq_starts=i32([p_last]), seq_new=i32([1]))
            ops.attention_decode_fused(qkv, inv, out, cache.k, cache.v, cache.table, step, H, KV, hd, scale, window, 3)
        else:
            _fill_cache(cache, 1, k, v)
            qbuf = q.view(new, H * hd).to(dt).to(DEV)
            if kernel in ("simt_f32", "simt_bf16"):
                ops.attention_simt(qbuf, H * hd, out, cache.k, cache.v, cache.table, i32([p_last]), i32([1]), 1, H, KV, hd, scale, window)
            elif kernel == "decode_split":
                ops.attention_decode(qbuf, H * hd, out, cache.k, cache.v, cache.table, i32([p_last]), i32([1]), 1, H, KV, hd, scale, window, 3)
            else:
                few = kernel == "mma_decode"
                ops.attention_mma(qbuf, H * hd, out, cache.k, cache.v, cache.table, i32([0, new]), i32([1]), i32([n - new]), i32([new]),
                                  1, new, new, H, KV, hd, scale, window, 3 if few else 1, few)
        ops.check_status(out.device)
        kk, vv = k.to(dt).float(), v.to(dt).float()
        for j in range(new):
            pos = n - new + j
            qv = q[j].to(dt).float()
            ref = _ref_attention(qv, kk, vv, pos, scale, window)
            inside = pos - window + 1 <= edge <= pos
            if inside:                                          # the reference itself is the edge key's value then
                assert float((ref - vv[edge].double().repeat_interleave(H // KV, dim=0)).abs().max()) < 1e-6
            _close(out[j].view(H, hd), ref, name, f"{kernel}: dominant key at {edge}, query at {pos}, window {window}",
                   scale=float(vv.abs().max()))


@pytest.mark.parametrize("M,I,K", [(1, 64, 64), (8, 512, 192), (33, 14336 // 8, 4096 // 8), (64, 128, 72), (65, 512, 192),
                                   (96, 1792, 520), (128, 256, 4096), (200, 448, 136), (256, 2560, 2048), (257, 512, 192),
                                   (300, 1792, 520), (2048, 256, 4096), (2048, 2560, 2048), (1100, 1792, 520)])
def test_gate_up_product_with_swiglu_epilogue(ops, M, I, K):
    torch.manual_seed(18)
    x = torch.randn(M, K, device=DEV).bfloat16()
    gate = (torch.randn(I, K, device=DEV) * 0.05).bfloat16()
    up = (torch.randn(I, K, device=DEV) * 0.05).bfloat16()
    assert ops.swiglu_fusable(K, I, torch.bfloat16)
    w = ops.interleave_gate_up(gate, up)
    assert torch.equal(w[64:128], up[:64]) and torch.equal(w[128:192], gate[64:128]) if I > 64 else True
    out = torch.full((M, I), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.matmul_swiglu(x, w, out)
    ops.check_status(out.device)
    g = x.double().cpu() @ gate.double().cpu().T
    u = x.double().cpu() @ up.double().cpu().T
    ref = g / (1 + torch.exp(-g)) * u
    err = float((out.double().cpu() - ref).abs().max())
    assert err <= 8e-3 * float(ref.abs().max()) + 1e-6, f"fused swiglu {M}x{I}x{K}: error {err:.3e}"


# the cases with 7 * KV * splits > 444 take the light CTAs (two warps, half pages) of the head size 128
@pytest.mark.parametrize("H,KV,hd,window,splits,pieces", [(8, 2, 128, 0, 1, 0), (32, 8, 128, 0, 5, 6), (4, 4, 64, 0, 3, 2),
                                                          (6, 2, 64, 0, 16, 0), (8, 8, 128, 100, 2, 3), (16, 1, 128, 0, 4, 1),
                                                          (32, 8, 128, 0, 9, 6), (8, 8, 128, 100, 8, 0), (64, 64, 128, 0, 2, 1),
                                                          (24, 8, 128, 33, 16, 9), (64, 8, 128, 0, 9, 3),
                                                          (32, 8, 128, 0, 12, 6), (8, 8, 128, 100, 11, 0), (48, 16, 128, 0, 7, 2)])
def test_attention_decode_fused(ops, H, KV, hd, window, splits, pieces):
    """Rotation of q and k, the cache write, attention and the split merge in one kernel, against
    the separate rotary kernel followed by the reference attention; twice, so that the counters
    the kernel leaves behind are shown to be zero again."""
    from types import SimpleNamespace
    seqs = [(199, 1), (0, 1), (64, 1), (128, 1), (63, 1), (249, 1), (1000, 1)]
    cache, slots, ks, vs, qbuf, stride, cu, sl, st, nw, rows = _ragged_problem(H, KV, hd, seqs, seed=19)
    inv = plain_llama.rope_inverse_frequencies(hd, 500000.0, None).to(DEV)
    scale = 1 / math.sqrt(hd)
    for round_ in range(2):
        torch.manual_seed(20 + round_)
        qkv = torch.randn(rows, stride, device=DEV).bfloat16()
        step = SimpleNamespace(n_seqs=rows, n_tokens=rows, is_decode=True, cu_tokens=cu, seq_slots=sl, seq_starts=st, seq_new=nw)
        arg = qkv
        if pieces:
            parts = torch.randn(pieces, rows, stride, device=DEV)
            parts[-1] = qkv.float() - parts[:-1].sum(0)
            arg = parts.contiguous()
            exact = parts[0].clone()
            for z in range(1, pieces):
                exact += parts[z]
        else:
            exact = qkv.float()
        out = torch.full((rows, H * hd), 3.0, device=DEV, dtype=torch.bfloat16)
        ops.attention_decode_fused(arg, inv, out, cache.k, cache.v, cache.table, step, H, KV, hd, scale, window, splits)
        e = exact.cpu().view(rows, H + 2 * KV, hd)
        for i, (s0, _) in enumerate(seqs):
            p = torch.tensor([s0])
            qr = plain_llama.rope_rotate(e[i:i + 1, :H], p, inv.cpu())[0].bfloat16().float()
            kr = plain_llama.rope_rotate(e[i:i + 1, H:H + KV], p, inv.cpu())[0]
            kk = torch.cat([ks[i][:s0], kr[None]], 0).bfloat16().float()
            vv = torch.cat([vs[i][:s0], e[i:i + 1, H + KV:]], 0).bfloat16().float()
            ref = _ref_attention(qr, kk, vv, s0, scale, window)
            _close(out[i].view(H, hd), ref, "bfloat16", f"fused decode seq {i} round {round_}", scale=float(vv.abs().max()))
            got_k = cache.rows("k", slots[i], s0 + 1)[s0]
            got_v = cache.rows("v", slots[i], s0 + 1)[s0]
            _close(got_k, kr, "bfloat16", f"new key of seq {i}", scale=float(e.abs().max()))
            _close(got_v, e[i, H + KV:], "bfloat16", f"new value of seq {i}", scale=float(e.abs().max()))
    assert int(ops._zero_counters(torch.device(DEV), 1).abs().sum()) == 0


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("H,KV", [(8, 2), (32, 8), (4, 4), (6, 2), (8, 1), (16, 1)])
def test_attention_tcgen05_prefill(ops, H, KV, hd):
    seqs = [(0, 150), (0, 1), (60, 70), (3, 64), (0, 65), (100, 5), (0, 300)]
    cache, slots, ks, vs, qbuf, stride, cu, sl, st, nw, rows = _ragged_problem(H, KV, hd, seqs, seed=21)
    out = torch.full((rows + 2, H * hd), 3.0, device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    ops.attention_tcgen05(qbuf, stride, out, cache.k, cache.v, cache.table, cu, sl, st, nw, len(seqs), max(t for _, t in seqs),
                          rows, H, KV, hd, scale)
    ops.check_status(out.device)
    assert float((out[rows:].float() - 3.0).abs().max()) == 0.0, "a padding row was written"
    r = 0
    for i, (s0, t) in enumerate(seqs):
        kk, vv = ks[i].bfloat16().float(), vs[i].bfloat16().float()
        for j in range(t):
            qv = qbuf[r, :H * hd].float().cpu().view(H, hd)
            ref = _ref_attention(qv, kk, vv, s0 + j, scale, 0)
            _close(out[r].view(H, hd), ref, "bfloat16", f"tcgen05 prefill seq {i} token {j}", scale=float(vv.abs().max()))
            r += 1


@pytest.mark.parametrize("hd", [128, 64])
def test_attention_tcgen05_finds_one_far_key_among_thousands(ops, hd):
    torch.manual_seed(22)
    dt = torch.bfloat16
    H, KV, n, new = 8, 2, 3000, 40
    for far in (0, 63, 64, 127, 128, 1999, 2999):
        cache = Paged(2, 3072, KV, hd, dt, seed=7)
        k = torch.randn(n, KV, hd) * 0.1
        v = torch.randn(n, KV, hd)
        k[far] = 0
        k[far, :, 9] = 40.0
        _fill_cache(cache, 1, k, v)
        q = torch.randn(new, H, hd) * 0.1
        q[:, :, 9] = 40.0
        qbuf = q.view(new, H * hd).to(dt).to(DEV)
        out = torch.empty(new, H * hd, device=DEV, dtype=dt)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        ops.attention_tcgen05(qbuf, H * hd, out, cache.k, cache.v, cache.table, i32([0, new]), i32([1]), i32([n - new]), i32([new]),
                              1, new, new, H, KV, hd, 1 / math.sqrt(hd))
        ops.check_status(out.device)
        want = v[far].to(dt).float().repeat_interleave(H // KV, dim=0)
        for j in range(new):
            if far <= n - new + j:
                _close(out[j].view(H, hd), want, "bfloat16", f"far key at {far}, query {j}")


@pytest.mark.parametrize("M,N,K,splits", [(1, 128, 64, 1), (8, 4096, 4096, None), (16, 1000, 520, 3), (33, 384, 136, 2),
                                          (64, 640, 1024, 4), (5, 4096, 14336, None)])
def test_products_with_the_residual_stream_folded_in(ops, M, N, K, splits):
    """The two decode forms of the skinny product.  Consumer: activations are the stream's rows
    times the norm weight, and the epilogue multiplies row m by rsqrt(mean(x_m^2) + eps) from
    pieces of sum(x^2): the product of the normalised rows.  Producer: the result is added into a
    residual stream by the last CTA of every column tile, which also returns the pieces of the
    new rows' sums of squares and the new rows times the next norm's weight.  Twice, to show the
    counters are left at zero."""
    torch.manual_seed(23)
    eps = 1e-5
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    for round_ in range(2):
        x = torch.randn(M, K, device=DEV) * 2
        nw = 1 + 0.1 * torch.randn(K, device=DEV)
        pieces = 3
        ss = torch.zeros(pieces, 64, device=DEV)
        full = (x * x).sum(1)
        ss[0, :M] = full * 0.25
        ss[1, :M] = full * 0.5
        ss[2, :M] = full - ss[0, :M] - ss[1, :M]
        scaled = (x * nw).bfloat16()
        inv = torch.rsqrt((x.double() ** 2).mean(1) + eps).cpu()
        ref = (scaled.double().cpu() * inv[:, None]) @ w.double().cpu().T
        # the same thing is the product of the normalised rows, up to the rounding of the rows
        normed = plain_llama.rmsnorm(x.cpu(), nw.cpu(), eps).double() @ w.double().cpu().T
        assert float((ref - normed).abs().max()) <= 1e-2 * float(normed.abs().max())
        got = ops.gemm_skinny_stream(w, scaled, row_scale=(ss, eps), splits=splits)
        ops.check_status(torch.device(DEV))
        err = float((got.sum(0).double().cpu() - ref).abs().max())
        assert err <= 1e-4 * float(ref.abs().max()) + 1e-5, f"product with 1 / rms in the epilogue {M}x{N}x{K}: {err:.3e}"
        # the same product added into a stream
        a = (scaled.float() * inv.float().to(DEV)[:, None]).bfloat16()
        ref_a = a.double().cpu() @ w.double().cpu().T
        sink = torch.randn(M, N, device=DEV)
        next_w = 1 + 0.1 * torch.randn(N, device=DEV)
        before = sink.clone()
        ss_out, scaled_out = ops.gemm_skinny_stream(w, a, sink=(sink, next_w), splits=splits)
        ops.check_status(torch.device(DEV))
        want = before.double().cpu() + ref_a
        err = float((sink.double().cpu() - want).abs().max())
        assert err <= 1e-4 * float(ref_a.abs().max()) + 1e-5, f"product added into the stream {M}x{N}x{K}: {err:.3e}"
        got_ss = ss_out[:, :M].sum(0).double().cpu()
        want_ss = (sink.double().cpu() ** 2).sum(1)
        assert float(((got_ss - want_ss) / want_ss).abs().max()) < 1e-5, "sums of squares of the new rows"
        assert torch.equal(scaled_out, (sink * next_w).bfloat16()), "the new rows times the next norm's weight"
        only_ss, none = ops.gemm_skinny_stream(w, a, sink=(before.clone(), None), splits=splits)
        assert none is None and torch.equal(only_ss[:, :M], ss_out[:, :M])
    if N % 128 == 0 and K % 8 == 0:
        gate = (torch.randn(N // 2, K, device=DEV) * 0.05).bfloat16()
        up = (torch.randn(N // 2, K, device=DEV) * 0.05).bfloat16()
        if (N // 2) % 64 == 0:
            act = ops.gemm_skinny_stream(ops.interleave_gate_up(gate, up), scaled, row_scale=(ss, eps), swiglu=True)
            rows = scaled.double().cpu() * inv[:, None]
            g = rows @ gate.double().cpu().T
            u = rows @ up.double().cpu().T
            r = g / (1 + torch.exp(-g)) * u
            assert float((act.double().cpu() - r).abs().max()) <= 8e-3 * float(r.abs().max()) + 1e-6
    assert int(ops._zero_counters(torch.device(DEV), 1, "gemm").abs().sum()) == 0

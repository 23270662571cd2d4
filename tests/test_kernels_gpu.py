"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda")


def kernels():
    from cisr_b200.ops import kernels as k
    return k


def close(a, b, atol, rtol, what=""):
    torch.testing.assert_close(a.double().cpu(), b.double().cpu(), atol=atol, rtol=rtol, msg=lambda m: f"{what}: {m}")


def product_rounding_sigma(a, w):
    """An upper bound on the standard deviation of (bfloat16-rounded a) @ w^T around a @ w^T, per output element, for
    float64 `a` [m, k] and `w` [n, k].  Rounding a_k to eight significant bits moves it by at most half a unit in the
    last place, uniformly: a standard deviation of 2^-8 / sqrt(3) times the power of two below |a_k|, so at most that
    times |a_k| itself, wherever in the computation of `a` the rounding happens (before or after a common factor).
    The errors are independent, so the variance of a sum is the sum of (2^-8 a_k w_k)^2 / 3."""
    return (2.0 ** -8 / 3 ** 0.5) * torch.sqrt((a * a) @ (w * w).T)


def within(out, ref, bound, what):
    """|out - ref| <= bound element by element (all float64 on the CPU), with the worst offender in the message."""
    excess = (out.double().cpu() - ref).abs() - bound
    worst = int(excess.argmax())
    assert excess.max() <= 0, (f"{what}: element {worst} is off by {float((out.double().cpu() - ref).abs().flatten()[worst]):.3e}, "
                               f"bound {float(bound.flatten()[worst]):.3e}")


@pytest.mark.parametrize("hidden", [10, 64, 130, 200, 576, 1000, 2048, 4096, 5000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(hidden, dtype):
    k = kernels()
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(7, hidden, generator=g) * 3
    delta = torch.randn(7, hidden, generator=g)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    eps = 3e-6
    xd, dd = x.to(dev()), delta.to(dev())
    out = torch.empty(7, hidden, dtype=dtype, device=dev())
    k.add_rmsnorm(xd, dd, w.to(dev()), eps, out)
    ref_x = x.double() + delta.double()
    ref = pl.rms_norm(ref_x, w.double(), eps)
    close(xd, ref_x, 1e-6, 1e-6, "residual sum")
    if dtype == torch.float32:
        close(out, ref, 2e-6, 2e-6, "norm")
    else:
        close(out, ref, 0, 2 ** -8, "norm rounded once to bfloat16")
    # selected rows, no delta, nothing written back
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=dev())
    before = xd.clone()
    out2 = torch.empty(3, hidden, dtype=torch.float32, device=dev())
    k.add_rmsnorm(xd, None, w.float().to(dev()), eps, out2, rows=rows, write_back=False)
    assert torch.equal(xd, before)
    close(out2, pl.rms_norm(ref_x[[5, 0, 5]], w.double(), eps), 3e-6, 3e-6, "selected rows")
    zero = torch.zeros(2, hidden, device=dev())
    outz = torch.ones(2, hidden, device=dev())
    k.add_rmsnorm(zero, None, w.float().to(dev()), eps, outz)
    assert torch.equal(outz, torch.zeros_like(outz))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_swiglu(dtype):
    k = kernels()
    g = torch.Generator().manual_seed(3)
    table = torch.randn(301, 70, generator=g).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 70, device=dev())
    k.embedding(table.to(dev()), ids.to(dev()), out)
    assert torch.equal(out.cpu(), pl.embed(table, ids.tolist()).float())
    gate_up = torch.randn(9, 2 * 333, generator=g) * 4
    gate_up[0, 0], gate_up[0, 1] = 90.0, -90.0            # far tails of the sigmoid stay finite
    act = torch.empty(9, 333, dtype=dtype, device=dev())
    k.swiglu(gate_up.to(dev()), act)
    gt, up = gate_up[:, :333].double(), gate_up[:, 333:].double()
    ref = gt / (1 + torch.exp(-gt)) * up
    assert torch.isfinite(act).all()
    close(act, ref, 1e-6 if dtype == torch.float32 else 1e-30, 3e-6 if dtype == torch.float32 else 2 ** -8, "swiglu")


@pytest.mark.parametrize("m,n,kk", [(1, 7, 13), (5, 576, 64), (33, 100, 257), (64, 3072, 576), (130, 49, 1536)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm(m, n, kk, dtype):
    k = kernels()
    g = torch.Generator().manual_seed(m * n)
    a = torch.randn(m, kk, generator=g).to(dtype)
    w = torch.randn(n, kk, generator=g).to(dtype)
    out = torch.empty(m, n, device=dev())
    k.gemm(a.to(dev()), w.to(dev()), out)
    ref = a.double() @ w.double().T
    # float32: the library's blocked sums stay within 2e-6 * sqrt(K).  bfloat16 products are exact in float, so the
    # error is that of adding K unit-size terms one k-block after the other in float: a partial sum of size ~sqrt(i)
    # rounds to 6e-8 of itself at every step, about 6e-8 * K / sqrt(2) in all (one standard deviation); four of those.
    atol = 2e-6 * math.sqrt(kk) if dtype == torch.float32 else max(2e-6 * math.sqrt(kk), 4 * 6e-8 * kk / math.sqrt(2))
    close(out, ref, atol, 1e-5, f"gemm {m}x{n}x{kk}")


def test_float32_products_are_true_32_bit():
    """A reduced-precision matrix mode (TF32 keeps 10 mantissa bits) would lose the small term below."""
    k = kernels()
    a = torch.tensor([[1.0, 2.0 ** -12] + [0.0] * 62], device=dev())
    w = torch.tensor([[1.0, 1.0] + [0.0] * 62] * 8, device=dev())
    out = torch.empty(1, 8, device=dev())
    k.gemm(a, w, out)
    assert out[0, 0].item() == 1.0 + 2.0 ** -12


def paged(k_dense, v_dense, page_size, n_pages, seed, dtype):
    """Scatter dense [T, Hkv, D] keys and values into shuffled pages; returns caches and a table row."""
    t, hkv, d = k_dense.shape
    need = -(-t // page_size)
    perm = np.random.default_rng(seed).permutation(n_pages)[:need]
    kc = torch.full((n_pages, hkv, page_size, d), float("nan"), dtype=dtype)
    vc = torch.full((n_pages, hkv, page_size, d), float("nan"), dtype=dtype)
    for pos in range(t):
        page, off = perm[pos // page_size], pos % page_size
        kc[page, :, off] = k_dense[pos].to(dtype)
        vc[page, :, off] = v_dense[pos].to(dtype)
    return kc, vc, perm.astype(np.int32)


def run_attention(q_all, k_all, v_all, q_lens, page_size, dtype, window=None, split_size=None, seed=0, width=64, kind="auto",
                  staging="auto", fill=0.0, wide=False):
    """Requests given as whole sequences; the last q_lens[r] positions of each are this step's queries.
    Cache rows that no request has written hold `fill`."""
    k = kernels()
    R = len(q_all)
    hq, d = q_all[0].shape[1:]
    hkv = k_all[0].shape[1]
    n_pages = sum(-(-x.shape[0] // page_size) for x in k_all) + 3
    kc = torch.full((n_pages, hkv, page_size, d), fill, dtype=dtype)
    vc = torch.full_like(kc, fill)
    table = np.full((R + 1, width), -1, dtype=np.int32)
    perm = np.random.default_rng(seed).permutation(n_pages)
    used = 0
    for r in range(R):
        t = k_all[r].shape[0]
        need = -(-t // page_size)
        pages = perm[used:used + need]; used += need
        table[r + 1, :need] = pages                      # request r sits in slot r + 1
        for pos in range(t):
            kc[pages[pos // page_size], :, pos % page_size] = k_all[r][pos].to(dtype)
            vc[pages[pos // page_size], :, pos % page_size] = v_all[r][pos].to(dtype)
    q = torch.cat([q_all[r][-q_lens[r]:] for r in range(R)]).to(dtype)
    total = q.shape[0]
    q_start = np.cumsum([0] + q_lens[:-1]).astype(np.int32)
    ctx = np.asarray([x.shape[0] for x in k_all], dtype=np.int32)
    tile_req, tile_q0, dec_req = [], [], []
    for r, n in enumerate(q_lens):
        if n == 1:
            dec_req.append(r)
        else:
            for q0 in range(0, n, k.PREFILL_TILE):
                tile_req.append(r); tile_q0.append(q0)
    i32 = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=dev())
    out = torch.full((total, hq, d), float("nan"), dtype=dtype, device=dev())
    args = dict(hq=hq, hkv=hkv, page_size=page_size, scale=d ** -0.5, window=window, kind=kind)
    kcd, vcd, qd = kc.to(dev()), vc.to(dev()), q.to(dev()).contiguous()
    req_slot = i32(np.arange(1, R + 1)); tab = i32(table)
    if tile_req and wide:       # the tcgen05 kernel: tiles of 128 queries
        wide_req, wide_q0 = [], []
        for r, n in enumerate(q_lens):
            if n > 1:
                for q0 in reversed(range(0, n, k.WIDE_TILE)):
                    wide_req.append(r); wide_q0.append(q0)
        k.attn_prefill_wide(qd, out, kcd, vcd, req_slot, tab, i32(wide_req), i32(wide_q0), i32(q_start), i32(q_lens), i32(ctx),
                            hq, hkv, page_size, d ** -0.5, window)
    elif tile_req:
        k.attn_prefill(qd, out, kcd, vcd, req_slot, tab, i32(tile_req), i32(tile_q0), i32(q_start), i32(q_lens), i32(ctx), **args)
    if dec_req:
        max_ctx = int(max(ctx[r] for r in dec_req))
        size = split_size or 64
        n_splits = -(-max_ctx // size)
        partial = torch.full((len(dec_req), hq, n_splits, d), float("nan"), device=dev())
        stats = torch.full((len(dec_req), hq, n_splits, 2), float("nan"), device=dev())
        k.attn_decode(qd, out, kcd, vcd, req_slot, tab, i32(dec_req), len(dec_req), i32(q_start), i32(ctx), partial, stats,
                      split_size=size, n_splits=n_splits, staging=staging, **args)
    refs = []
    for r in range(R):
        qq = q_all[r].to(dtype).double(); kk = k_all[r].to(dtype).double(); vv = v_all[r].to(dtype).double()
        refs.append(pl.causal_attention(qq, kk, vv, window)[-q_lens[r]:])
    return out, torch.cat(refs)


def random_qkv(t, hq, hkv, d, seed, sharp=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(t, hq, d, generator=g) * sharp, torch.randn(t, hkv, d, generator=g), torch.randn(t, hkv, d, generator=g))


ATT_TOL = {torch.float32: (3e-6, 1e-5), torch.bfloat16: (2e-2, 2e-2)}


@pytest.mark.parametrize("d,hq,hkv", [(64, 9, 3), (128, 4, 4), (48, 5, 1), (16, 2, 2), (32, 40, 2), (144, 2, 1)])
@pytest.mark.parametrize("dtype,kind", [(torch.float32, "auto"), (torch.bfloat16, "auto"), (torch.bfloat16, "simt")])
def test_attention_mixed_portions_and_decode(d, hq, hkv, dtype, kind):
    """Whole prompts, portions with earlier context, and single tokens in one launch pair; pages of 8 in shuffled order.
    bfloat16 runs on the tensor cores ("auto", heads up to 128 wide) and on the CUDA cores ("simt")."""
    lens, q_lens = [200, 77, 130, 1, 301, 65], [200, 13, 1, 1, 1, 2]
    data = [random_qkv(t, hq, hkv, d, 10 * d + i, sharp=2.0) for i, t in enumerate(lens)]
    out, ref = run_attention([x[0] for x in data], [x[1] for x in data], [x[2] for x in data], q_lens, 8, dtype, seed=d, kind=kind)
    assert torch.isfinite(out).all()
    close(out, ref, *ATT_TOL[dtype], "attention")


@pytest.mark.parametrize("d,hq,hkv", [(64, 9, 3), (128, 8, 2), (64, 40, 2)])
@pytest.mark.parametrize("page_size", [8, 16, 64, 128])
@pytest.mark.parametrize("staging,clusters", [("tensor_map", True), ("tensor_map", False), ("gather", False)])
def test_decode_attention_by_tensor_map_copies_and_by_gather(d, hq, hkv, page_size, staging, clusters):
    """Single tokens over contexts at tile, page and key-range edges, with both ways of staging the tiles.  Cache rows
    that nobody wrote hold NaN: a value row beyond the newest key must not reach the output through a zero weight.
    Forty query heads on two key heads take two launches of sixteen and four rows.  Ranges of 192 keys: eleven, merged
    in one thread-block cluster; of 64: thirty-three, three clusters of eleven and the merge kernel; clusters off:
    every range through the merge kernel."""
    k = kernels()
    lens = [1, 63, 64, 65, 200, 449, 512, 1000, 2100]
    data = [random_qkv(t, hq, hkv, d, 7 * d + i, sharp=2.0) for i, t in enumerate(lens)]
    k.set_clusters(clusters)
    try:
        for window, split_size in ((None, 192), (100, 192), (None, 64)):
            out, ref = run_attention([x[0] for x in data], [x[1] for x in data], [x[2] for x in data], [1] * len(lens), page_size,
                                     torch.bfloat16, window=window, split_size=split_size, seed=d + page_size, width=272,
                                     staging=staging, fill=float("nan"))
            assert torch.isfinite(out).all()
            close(out, ref, *ATT_TOL[torch.bfloat16], f"decode attention, {staging}, window {window}, ranges of {split_size}")
    finally:
        k.set_clusters(False)


@pytest.mark.parametrize("d,hq,hkv", [(64, 9, 3), (128, 4, 2), (64, 2, 2)])
@pytest.mark.parametrize("page_size", [8, 16, 128, 256])
@pytest.mark.parametrize("window", [None, 100])
def test_prompt_attention_on_tcgen05(d, hq, hkv, page_size, window):
    """Whole prompts and portions with earlier context in one launch: lengths at and around the 128-query and 128-key
    tile edges, one longer than three tiles; cache rows that nobody wrote hold NaN (a value row beyond the last key
    must not reach the output through a zero weight).  Single tokens in the same step go to the decode kernel."""
    lens, q_lens = [200, 77, 130, 128, 301, 129, 515, 1], [200, 13, 2, 128, 44, 129, 515, 1]
    data = [random_qkv(t, hq, hkv, d, 11 * d + i, sharp=2.0) for i, t in enumerate(lens)]
    out, ref = run_attention([x[0] for x in data], [x[1] for x in data], [x[2] for x in data], q_lens, page_size, torch.bfloat16,
                             window=window, seed=d + page_size, width=128, fill=float("nan"), wide=True)
    assert torch.isfinite(out).all()
    close(out, ref, *ATT_TOL[torch.bfloat16], f"tcgen05 prompt attention, pages of {page_size}, window {window}")


@pytest.mark.parametrize("needle", [0, 127, 128, 255, 256, 600])
def test_prompt_attention_on_tcgen05_finds_one_far_key(needle):
    """One key is made to stand out for the last query of a 700-token prompt: the output must be that key's value."""
    t, hq, hkv, d = 700, 6, 2, 64
    q, k_, v = random_qkv(t, hq, hkv, d, needle)
    q[-1] = q[-1] / q[-1].norm(dim=-1, keepdim=True) * 6
    for h in range(hkv):
        k_[needle, h] = q[-1, h * 3] * 4
    v[needle] = 100.0
    out, ref = run_attention([q], [k_], [v], [t], 16, torch.bfloat16, seed=needle, wide=True)
    close(out, ref, 0.5, 2e-2, f"needle at {needle}")
    assert out[-1, 0, 0].item() > 99.0 and out[-1, 3, 0].item() > 99.0


def test_tensor_map_staging_refuses_what_it_cannot_take():
    k = kernels()
    i32 = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=dev())
    for d, page, split in ((48, 16, 64), (64, 12, 64), (64, 16, 100)):
        q = torch.zeros(1, 2, d, dtype=torch.bfloat16, device=dev())
        kc = torch.zeros(4, 1, page, d, dtype=torch.bfloat16, device=dev())
        partial = torch.empty(1, 2, 2, d, device=dev()); stats = torch.empty(1, 2, 2, 2, device=dev())
        with pytest.raises(k.KernelError, match="tensor-map staging"):
            k.attn_decode(q, torch.empty_like(q), kc, kc.clone(), i32([0]), i32(np.zeros((1, 8))), i32([0]), 1, i32([0]), i32([5]),
                          partial, stats, 2, 1, page, d ** -0.5, None, split, 2, staging="tensor_map")


@pytest.mark.parametrize("needle", [0, 15, 16, 63, 64, 255, 256, 511, 640])
@pytest.mark.parametrize("q_len", [1, 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds(needle, q_len, dtype):
    """One key is made to stand out for the last query; the output must be that key's value (page and split edges)."""
    t, hq, hkv, d = 700, 6, 2, 64
    q, k_, v = random_qkv(t, hq, hkv, d, needle)
    q[-1] = q[-1] / q[-1].norm(dim=-1, keepdim=True) * 6
    for h in range(hkv):
        k_[needle, h] = q[-1, h * 3] * 4          # aligned with the first query head of each group
    v[needle] = 100.0
    out, ref = run_attention([q], [k_], [v], [q_len], 16, dtype, split_size=64, seed=needle)
    close(out, ref, 2e-4 if dtype == torch.float32 else 0.5, 1e-5 if dtype == torch.float32 else 2e-2, f"needle at {needle}")
    assert out[-1, 0, 0].item() > 99.0 and out[-1, 3, 0].item() > 99.0


@pytest.mark.parametrize("window", [1, 16, 17, 100])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_window_edge(window, dtype):
    """Keys at the window's edge are made large: one position too many or too few changes the result visibly."""
    t, hq, hkv, d = 260, 4, 2, 32
    q, k_, v = random_qkv(t, hq, hkv, d, window)
    for pos in (t - 1 - window, t - window, 40 - window, 41 - window):
        if pos >= 0:
            v[pos] = 50.0 * (1 + pos % 3)
    lens_q = [[t], [1], [t - 40]]
    for q_lens in lens_q:
        out, ref = run_attention([q], [k_], [v], q_lens, 16, dtype, window=window, seed=window)
        close(out, ref, 5e-5 if dtype == torch.float32 else 0.3, 1e-5 if dtype == torch.float32 else 2e-2, f"window {window}")


@pytest.mark.parametrize("dtype,d", [(torch.float32, 16), (torch.bfloat16, 64)])
def test_attention_ignores_pages_that_the_window_has_passed(dtype, d):
    """Entries of passed pages are -1 in the table; the kernels must not follow them (bfloat16 heads of 64: the
    decode kernel that stages by tensor-map copies fetches such a page from beyond the cache, as zeros)."""
    k = kernels()
    t, hq, hkv, window, page = 100, 2, 1, 20, 8
    q, k_, v = random_qkv(t, hq, hkv, d, 5)
    q, k_, v = q.to(dtype).float(), k_.to(dtype).float(), v.to(dtype).float()
    kc, vc, pages = paged(k_, v, page, 20, 1, dtype)
    i32 = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=dev())
    for q_len in (1, 3):
        table = np.full((1, 16), -1, dtype=np.int32)
        table[0, :len(pages)] = pages
        dead = (t - q_len - window + 1) // page       # pages wholly before what the step's first query sees
        table[0, :dead] = -1
        out = torch.empty(q_len, hq, d, dtype=dtype, device=dev())
        common = (q[-q_len:].contiguous().to(dtype).to(dev()), out, kc.to(dev()), vc.to(dev()), i32([0]), i32(table))
        if q_len == 1:
            partial = torch.empty(1, hq, 2, d, device=dev()); stats = torch.empty(1, hq, 2, 2, device=dev())
            k.attn_decode(*common, i32([0]), 1, i32([0]), i32([t]), partial, stats, hq, hkv, page, d ** -0.5, window, 64, 2)
        else:
            k.attn_prefill(*common, i32([0]), i32([0]), i32([0]), i32([q_len]), i32([t]), hq, hkv, page, d ** -0.5, window)
        ref = pl.causal_attention(q.double(), k_.double(), v.double(), window)[-q_len:]
        close(out, ref, *ATT_TOL[dtype], "window with freed pages")


@pytest.mark.parametrize("interleaved,rot", [(False, 32), (True, 32), (False, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_store(interleaved, rot, dtype):
    """Rotation of q and k, and keys and values landing on the right page and offset."""
    k = kernels()
    t, hq, hkv, d, page, theta = 11, 3, 2, 32, 4, 25000.0
    g = torch.Generator().manual_seed(1)
    proj = torch.randn(t, (hq + 2 * hkv) * d, generator=g)
    positions = torch.tensor([5, 6, 7, 8, 0, 1, 2, 3, 40, 41, 42], dtype=torch.int32)
    token_req = torch.tensor([0] * 4 + [1] * 4 + [2] * 3, dtype=torch.int32)
    req_slot = torch.tensor([2, 0, 1], dtype=torch.int32)
    table = torch.full((3, 16), -1, dtype=torch.int32)
    table[2, :3] = torch.tensor([7, 3, 9]); table[0, :1] = 5; table[1, 10] = 1
    half = rot // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / rot)
    cos = torch.empty(t, half, device=dev()); sin = torch.empty(t, half, device=dev())
    k.rotary_tables(positions.to(dev()), inv.to(dev()), cos, sin)
    angle = positions.double()[:, None] * inv[None]
    close(cos, torch.cos(angle), 1e-7, 0, "cos table"); close(sin, torch.sin(angle), 1e-7, 0, "sin table")
    q_out = torch.empty(t, hq, d, dtype=dtype, device=dev())
    kc = torch.zeros(12, hkv, page, d, dtype=dtype, device=dev()); vc = torch.zeros_like(kc)
    k.rope_store(proj.to(dev()), hq * d, (hq + hkv) * d, cos, sin, half, interleaved, q_out, kc, vc, token_req.to(dev()),
                 positions.to(dev()), req_slot.to(dev()), table.to(dev()), page, hq, hkv, d)

    def rotate(x):
        x = x.double()
        out = x.clone()
        c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        if interleaved:
            a, b = x[..., 0:rot:2], x[..., 1:rot:2]
            out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, b * c + a * s
        else:
            a, b = x[..., :half], x[..., half:rot]
            out[..., :half], out[..., half:rot] = a * c - b * s, b * c + a * s
        return out

    if not interleaved and rot == d:
        close(rotate(proj[:, :hq * d].reshape(t, hq, d)), pl.rotary(proj[:, :hq * d].reshape(t, hq, d).double(), positions, theta), 1e-12, 0, "test's own rotation")
    tol = (2e-6, 2e-6) if dtype == torch.float32 else (0, 2 ** -8)
    close(q_out, rotate(proj[:, :hq * d].reshape(t, hq, d)), *tol, "q")
    k_ref = rotate(proj[:, hq * d:(hq + hkv) * d].reshape(t, hkv, d))
    v_ref = proj[:, (hq + hkv) * d:].reshape(t, hkv, d).double()
    written = 0
    for i in range(t):
        page_id = int(table[int(req_slot[int(token_req[i])]), int(positions[i]) // page])
        off = int(positions[i]) % page
        close(kc[page_id, :, off], k_ref[i], *tol, "k in cache"); close(vc[page_id, :, off], v_ref[i], *tol, "v in cache")
        written += 1
    assert int((kc.float().abs().sum(dim=(1, 3)) > 0).sum()) == written     # nothing else was touched


def test_table_update_and_page_copy():
    k = kernels()
    table = torch.full((4, 8), -1, dtype=torch.int32, device=dev())
    idx = torch.tensor([0, 9, 31, -1], dtype=torch.int32, device=dev())
    val = torch.tensor([5, 6, 7, 99], dtype=torch.int32, device=dev())
    k.table_update(table, idx, val)
    expect = torch.full((32,), -1, dtype=torch.int32); expect[0], expect[9], expect[31] = 5, 6, 7
    assert torch.equal(table.cpu().view(-1), expect)
    pool = torch.randn(3, 2, 6, 2, 4, 8, device=dev())            # [entries, k|v, pages, kv_heads, page, dim]
    before = pool.clone()
    pairs = torch.tensor([[1, 4], [0, 5]], dtype=torch.int32, device=dev())
    page_bytes = 2 * 4 * 8 * 4
    k.page_copy(pool, pairs, 6, 6 * page_bytes, page_bytes)
    assert torch.equal(pool[:, :, 4], before[:, :, 1]) and torch.equal(pool[:, :, 5], before[:, :, 0])
    assert torch.equal(pool[:, :, :4], before[:, :, :4])


def test_greedy_sampling_takes_the_lowest_index_on_ties():
    from cisr_b200.sampling import sample_tokens
    logits = torch.randn(5, 1000, device=dev())
    logits[0, 700] = logits[0, 300] = 50.0
    logits[1, 999] = 60.0
    logits[2, 0] = 60.0
    got = sample_tokens(logits).cpu().tolist()
    assert got[:3] == [300, 999, 0] and got[3:] == logits[3:].argmax(dim=-1).cpu().tolist()
    # a vocabulary that several CTAs share per row (and whose rows do not all start on a 16-byte boundary): ties and
    # maxima in different CTAs' shares, at their edges
    vocab = 40001
    logits = torch.randn(6, vocab, device=dev())
    logits[0, 39999] = logits[0, 100] = 50.0
    logits[1, vocab - 1] = 60.0
    logits[2, 13336] = logits[2, 13335] = 55.0
    logits[3, 26672] = 52.0
    got = sample_tokens(logits).cpu().tolist()
    assert got[:4] == [100, vocab - 1, 13335, 26672] and got[4:] == logits[4:].argmax(dim=-1).cpu().tolist()


@pytest.mark.parametrize("vocab", [5, 301, 40001, 49152, 128256])
def test_temperature_sampling_is_an_inverse_cdf_of_softmax(vocab):
    from cisr_b200.sampling import sample_tokens, uniform
    g = torch.Generator().manual_seed(vocab)
    rows = 64
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(dev())
    temp = torch.full((rows,), 0.8, device=dev()); temp[0] = 0.0
    seed = torch.arange(rows, dtype=torch.int64, device=dev()) * 7919 + 3
    counter = torch.arange(rows, dtype=torch.int32, device=dev())
    got = sample_tokens(logits, temp, seed, counter).cpu().tolist()
    again = sample_tokens(logits, temp, seed, counter).cpu().tolist()
    assert got == again and got[0] == int(logits[0].argmax())
    for r in range(1, rows):
        u = uniform(int(seed[r]), int(counter[r]))
        assert 0.0 <= u < 1.0
        cdf = torch.cumsum(pl.temperature_probabilities(logits[r].cpu(), 0.8), dim=0)
        lo = cdf[got[r] - 1].item() if got[r] else 0.0
        assert lo - 1e-5 <= u <= cdf[got[r]].item() + 1e-5, f"row {r}: token {got[r]} does not hold u={u}"
    us = [uniform(11, c) for c in range(2000)]
    assert abs(np.mean(us) - 0.5) < 0.03 and len(set(us)) > 1990
    # the batch does not matter: one row alone draws the same token
    alone = sample_tokens(logits[5:6].contiguous(), temp[5:6].contiguous(), seed[5:6].contiguous(), counter[5:6].contiguous())
    assert alone.cpu().tolist() == [got[5]]


def test_unsupported_head_size_is_refused_clearly():
    k = kernels()
    with pytest.raises(k.KernelError, match="multiples of 16"):
        k.attention_library(40, torch.float32)
    with pytest.raises(k.KernelError, match="multiples of 16"):
        k.attention_library(272, torch.bfloat16)


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("n,kk", [(100, 64), (576, 576), (49, 1536), (960, 240), (3000, 72), (5000, 1000)])
@pytest.mark.parametrize("kind", ["latency", "stream"])
def test_skinny_gemm_plain(m, n, kk, kind):
    """The weight-streaming products (a CTA per 16 rows; persistent CTAs fed by tensor-map copies) against a float64
    product, from activations and from the fused norm.  N and K that are no multiples of the tiles; K = 1000 ends in
    the middle of a 64-wide box."""
    k = kernels()
    if kind == "stream" and m > k.STREAM_MAX_TOKENS:
        pytest.skip("the streaming kernel takes up to 16 tokens")
    g = torch.Generator().manual_seed(m * n + kk)
    w = (0.1 * torch.randn(n, kk, generator=g)).to(torch.bfloat16)
    a = torch.randn(m, kk, generator=g).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), device=dev())
    k.skinny_gemm(w.to(dev()), m, act=a.to(dev()), epilogue=k.EPI_PLAIN, out=out, kind=kind)
    close(out, a.double() @ w.double().T, 2e-5 * math.sqrt(kk), 1e-5, "skinny plain")
    # the residual form: the product added to what the output holds, one float add per element
    stream = (10 * torch.randn(m, n, generator=g)).float()
    added = stream.clone().to(dev())
    k.skinny_gemm(w.to(dev()), m, act=a.to(dev()), epilogue=k.EPI_PLAIN, out=added, kind=kind, accumulate=True)
    assert torch.equal(added.cpu(), stream + out.cpu())
    if m <= k.SKINNY_NORM_MAX_TOKENS:
        x = torch.randn(m + 3, kk, generator=g) * 2
        delta = torch.randn(m + 3, kk, generator=g)
        nw = 1 + 0.1 * torch.randn(kk, generator=g)
        rows = torch.randperm(m + 3, generator=g)[:m].to(torch.int32)
        out2 = torch.full((m, n), float("nan"), device=dev())
        k.skinny_gemm(w.to(dev()), m, x=x.to(dev()), delta=delta.to(dev()), norm_w=nw.to(dev()), eps=1e-5, rows=rows.to(dev()),
                      epilogue=k.EPI_PLAIN, out=out2, kind=kind)
        # the kernel may round the normed row to bfloat16 before or after the row's common factor 1 / rms: six standard
        # deviations of either rounding around the unrounded product
        h = pl.rms_norm((x + delta).double()[rows.long()], nw.double(), 1e-5)
        ref = h @ w.double().T
        within(out2, ref, 6 * product_rounding_sigma(h, w.double()) + 1e-5 * (1 + ref.abs()), "skinny plain with norm prologue")


@pytest.mark.parametrize("m", [1, 7, 16, 40])
@pytest.mark.parametrize("inter,kk", [(176, 64), (1536, 576), (250, 96), (13, 40), (2504, 1000)])
@pytest.mark.parametrize("kind", ["latency", "stream"])
def test_skinny_gemm_swiglu_and_residual_output(m, inter, kk, kind):
    k = kernels()
    if kind == "stream" and (m > k.STREAM_MAX_TOKENS or inter % 8):
        pytest.skip("the streaming kernel takes up to 16 tokens and feature counts that are multiples of 8")
    g = torch.Generator().manual_seed(m + inter)
    w = (0.2 * torch.randn(2 * inter, kk, generator=g)).to(torch.bfloat16)
    x = torch.randn(m, kk, generator=g)
    delta = torch.randn(m, kk, generator=g)
    nw = (1 + 0.1 * torch.randn(kk, generator=g)).to(torch.bfloat16)
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=dev())
    exact = pl.rms_norm((x + delta).double(), nw.double(), 2e-6)
    h = exact.to(torch.bfloat16)
    if m <= k.SKINNY_NORM_MAX_TOKENS:
        x_out = torch.full_like(x, float("nan")).to(dev())
        xd = x.to(dev())
        k.skinny_gemm(w.to(dev()), m, x=xd, delta=delta.to(dev()), norm_w=nw.to(dev()), eps=2e-6, x_out=x_out,
                      epilogue=k.EPI_SWIGLU, out=act, kind=kind)
        close(x_out, x.double() + delta.double(), 1e-6, 1e-6, "residual sum written by CTA 0")
        assert torch.equal(xd.cpu(), x)                                   # the input stream is not touched
    else:
        k.skinny_gemm(w.to(dev()), m, act=h.to(dev()), epilogue=k.EPI_SWIGLU, out=act, kind=kind)
    # gate and up within six standard deviations of the activations' rounding (wherever in the norm it happens), carried
    # through silu(g) * u (|silu'| <= 1.1), plus the output's own rounding to bfloat16
    gu = exact @ w.double().T
    sigma = product_rounding_sigma(exact, w.double())
    gate, up = gu[:, :inter], gu[:, inter:]
    silu = gate / (1 + torch.exp(-gate))
    ref = silu * up
    bound = 6 * (1.1 * up.abs() * sigma[:, :inter] + silu.abs() * sigma[:, inter:]) + 2.0 ** -8 * ref.abs() + 1e-4
    within(act, ref, bound, "skinny swiglu")


def plain_rotated_projection(hbf, w, positions, token_req, req_slot, table, page, n_pages, hq, hkv, dim, rot, interleaved, theta):
    """What the fused q/k/v kernels must leave behind, in float64 from the bfloat16-rounded inputs: q [m, hq, dim] and the
    key and value caches [pages, hkv, page, dim] (zero where nothing is written).  Whole-head split-half rotation is
    plain_llama.rotary (runtime/reference.py:9-15); a partial or interleaved rotation, which the reference does not
    have, is the same turn of pair (i, i + rot/2) or (2i, 2i + 1) of the first `rot` coordinates."""
    import plain_llama as pl
    proj = hbf.double().cpu() @ w.double().cpu().T
    m = proj.shape[0]
    pos = positions.cpu().long()
    q = proj[:, :hq * dim].reshape(m, hq, dim)
    kk = proj[:, hq * dim:(hq + hkv) * dim].reshape(m, hkv, dim)
    vv = proj[:, (hq + hkv) * dim:].reshape(m, hkv, dim)

    def turn(x):
        if rot == dim and not interleaved:
            return pl.rotary(x, pos, theta)
        half = rot // 2
        inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / rot)
        angle = pos.double()[:, None] * inv[None, :]
        c, s_ = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        out = x.clone()
        if interleaved:
            a, b = x[..., 0:rot:2], x[..., 1:rot:2]
            out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s_, b * c + a * s_
        else:
            a, b = x[..., :half], x[..., half:rot]
            out[..., :half], out[..., half:rot] = a * c - b * s_, b * c + a * s_
        return out

    q, kk = turn(q), turn(kk)
    kc = torch.zeros(n_pages, hkv, page, dim, dtype=torch.float64); vc = torch.zeros_like(kc)
    slots, tab = req_slot.cpu().long(), table.cpu().long()
    for t in range(m):
        row = tab[slots[token_req[t].item()]]
        pg, off = row[pos[t] // page].item(), (pos[t] % page).item()
        kc[pg, :, off], vc[pg, :, off] = kk[t], vv[t]
    return q, kc, vc


def check_rotated_projection(results, reference):
    """results[0]: the separate kernels, results[1]: the fused kernel; both against the float64 reference (a bfloat16
    result is within half a unit in the last place of its value plus the product's rounding), then against each other."""
    for i, what in enumerate(("q", "k cache", "v cache")):
        for got, path in ((results[1][i], "fused"), (results[0][i], "separate")):
            assert float(got.abs().sum()) > 0
            torch.testing.assert_close(got.double(), reference[i], atol=2e-2, rtol=2e-2, msg=lambda s: f"{path} {what} against float64: {s}")
            assert torch.equal(got == 0, reference[i] == 0) or what == "q", f"{path} {what}: other cache places were written"
        torch.testing.assert_close(results[1][i], results[0][i], atol=2e-2, rtol=2e-2, msg=lambda s: f"{what}, fused against separate: {s}")


@pytest.mark.parametrize("m", [1, 8, 11, 30])
@pytest.mark.parametrize("dim,hq,hkv,rot,interleaved", [(64, 9, 3, 64, False), (16, 2, 2, 16, False), (48, 5, 1, 32, True), (128, 2, 1, 128, False),
                                                        (96, 3, 1, 96, True), (32, 4, 2, 32, False)])
@pytest.mark.parametrize("kind,hidden", [("latency", 96), ("stream", 96), ("stream", 128)])
def test_skinny_gemm_rope_matches_plain_and_the_separate_kernels(m, dim, hq, hkv, rot, interleaved, kind, hidden):
    """Fused q/k/v product + rotation + cache write against the float64 plain rotation of the float64 product, and
    against product -> rope_store on the same inputs.  (A width of whole 64-column groups makes the streaming kernel
    fetch a stage as one box.)"""
    k = kernels()
    if kind == "stream" and (m > k.STREAM_MAX_TOKENS or dim % 32 or rot != dim):
        pytest.skip("the streaming kernel takes up to 16 tokens, head sizes in steps of 32 and whole-head rotation")
    page, theta = 4, 10000.0
    g = torch.Generator().manual_seed(m * dim)
    w = (0.2 * torch.randn((hq + 2 * hkv) * dim, hidden, generator=g)).to(torch.bfloat16).to(dev())
    hbf = torch.randn(m, hidden, generator=g).to(torch.bfloat16).to(dev())
    positions = torch.randperm(40, generator=g)[:m].to(torch.int32).to(dev())
    token_req = (torch.arange(m) % 3).to(torch.int32).to(dev())
    req_slot = torch.tensor([2, 0, 1], dtype=torch.int32, device=dev())
    table = torch.arange(36, dtype=torch.int32).reshape(3, 12).to(dev())          # every (slot, logical page) its own page
    half = rot // 2
    inv = (theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / rot)).to(dev())
    cos = torch.empty(m, half, device=dev()); sin = torch.empty(m, half, device=dev())
    k.rotary_tables(positions, inv, cos, sin)
    results = []
    for fused in (False, True):
        q = torch.zeros(m, hq, dim, dtype=torch.bfloat16, device=dev())
        kc = torch.zeros(36, hkv, page, dim, dtype=torch.bfloat16, device=dev()); vc = torch.zeros_like(kc)
        if fused:
            k.skinny_gemm(w, m, act=hbf, epilogue=k.EPI_ROPE, kind=kind,
                          rope=dict(cos=cos, sin=sin, rot_half=half, interleaved=interleaved, q_out=q, k_cache=kc, v_cache=vc,
                                    positions=positions, token_req=token_req, req_slot=req_slot, block_table=table, page_size=page,
                                    hq=hq, hkv=hkv, dim=dim))
        else:
            proj = torch.empty(m, w.shape[0], device=dev())
            k.gemm_library(hbf, w, proj)
            k.rope_store(proj, hq * dim, (hq + hkv) * dim, cos, sin, half, interleaved, q, kc, vc, token_req, positions, req_slot,
                         table, page, hq, hkv, dim)
        results.append((q.float().cpu(), kc.float().cpu(), vc.float().cpu()))
    check_rotated_projection(results, plain_rotated_projection(hbf, w, positions, token_req, req_slot, table, page, 36, hq, hkv, dim,
                                                               rot, interleaved, theta))


@pytest.mark.parametrize("m,n,kk", [(128, 128, 64), (128, 64, 128), (2048, 960, 576), (300, 576, 1536), (130, 49, 72),
                                    (257, 3072, 576), (129, 100, 8), (1000, 1000, 1000), (17, 960, 576), (64, 576, 1536),
                                    (2048, 576, 576), (100, 200, 4096)])
def test_gemm_tcgen05(m, n, kk):
    """The tcgen05 + TMA product against a float64 product, at sizes with ragged edges in M, N and K; grids of 128 x 256
    tiles, of 128 x 128 tiles, and of fewer tiles than SMs (deep rings of 128 x 128 and of 128 x 64 tiles); fewer tokens
    than a tile has rows."""
    k = kernels()
    g = torch.Generator().manual_seed(m + n + kk)
    a = torch.randn(m, kk, generator=g).to(torch.bfloat16)
    w = torch.randn(n, kk, generator=g).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), device=dev())
    k.gemm_tcgen05(a.to(dev()), w.to(dev()), out)
    k.raise_if_kernel_gave_up()
    ref = a.double() @ w.double().T
    close(out, ref, 2e-6 * kk ** 0.5 * 4, 1e-5, f"tcgen05 gemm {m}x{n}x{kk}")


@pytest.mark.parametrize("m,n,kk", [(2048, 576, 576), (300, 576, 1536), (130, 49, 72), (17, 960, 576), (1000, 1000, 1000)])
def test_gemm_tcgen05_adds_into_the_residual_stream(m, n, kk):
    """out += a w^T as the product's epilogue: every element is the one float sum of what was there and the product."""
    k = kernels()
    g = torch.Generator().manual_seed(m * n + kk)
    a = torch.randn(m, kk, generator=g).to(torch.bfloat16)
    w = torch.randn(n, kk, generator=g).to(torch.bfloat16)
    x = (10 * torch.randn(m, n, generator=g)).float()
    product = torch.empty((m, n), device=dev())
    k.gemm_tcgen05(a.to(dev()), w.to(dev()), product)
    out = x.clone().to(dev())
    k.gemm_tcgen05(a.to(dev()), w.to(dev()), out, accumulate=True)
    k.raise_if_kernel_gave_up()
    assert torch.equal(out.cpu(), x + product.cpu())             # the same bits as adding the product afterwards
    close(out, x.double() + a.double() @ w.double().T, 2e-6 * kk ** 0.5 * 4 + 1e-5, 1e-5, f"tcgen05 gemm + residual {m}x{n}x{kk}")


@pytest.mark.parametrize("m,inter,kk", [(128, 64, 64), (300, 176, 64), (2048, 1536, 576), (130, 250, 96), (129, 13, 40),
                                        (40, 96, 64), (64, 1536, 576), (1024, 4000, 128), (17, 1536, 576), (33, 250, 96),
                                        (100, 8192, 2048), (64, 14336, 4096)])
def test_gemm_tcgen05_swiglu_epilogue(m, inter, kk):
    k = kernels()
    g = torch.Generator().manual_seed(m + inter)
    a = torch.randn(m, kk, generator=g).to(torch.bfloat16)
    # a scale of 0.2 up to K = 576; beyond, the scale that keeps gate and up values at the size they have at K = 576
    w = (0.2 * min(1.0, math.sqrt(576 / kk)) * torch.randn(2 * inter, kk, generator=g)).to(torch.bfloat16)
    out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=dev())
    k.gemm_tcgen05_swiglu(a.to(dev()), w.to(dev()), out)
    k.raise_if_kernel_gave_up()
    gu = a.double() @ w.double().T
    ref = gu[:, :inter] / (1 + torch.exp(-gu[:, :inter])) * gu[:, inter:]
    close(out, ref, 1e-3, 2 ** -7, "tcgen05 swiglu epilogue")


@pytest.mark.parametrize("m", [17, 64, 128, 333, 2048])
@pytest.mark.parametrize("dim,hq,hkv", [(64, 9, 3), (128, 2, 1), (64, 2, 2), (128, 32, 8)])
def test_gemm_tcgen05_rope_epilogue_matches_plain_and_the_separate_kernels(m, dim, hq, hkv):
    """The tcgen05 q/k/v product with rotation and cache write as its epilogue against float64 (plain_llama.rotary of the
    float64 product), and against the library product followed by the rotate kernel."""
    k = kernels()
    hidden, page, theta = 96, 16, 10000.0
    g = torch.Generator().manual_seed(m + dim)
    w = (0.2 * torch.randn((hq + 2 * hkv) * dim, hidden, generator=g)).to(torch.bfloat16).to(dev())
    hbf = torch.randn(m, hidden, generator=g).to(torch.bfloat16).to(dev())
    positions = torch.arange(m, dtype=torch.int32).to(dev()) % 200
    n_req = -(-m // 200)
    token_req = (torch.arange(m) // 200).to(torch.int32).to(dev())               # requests of 200 tokens
    req_slot = torch.arange(n_req - 1, -1, -1, dtype=torch.int32).to(dev())
    table = torch.arange(16 * n_req, dtype=torch.int32).reshape(n_req, 16).to(dev())
    half = dim // 2
    inv = (theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / dim)).to(dev())
    cos = torch.empty(m, half, device=dev()); sin = torch.empty(m, half, device=dev())
    k.rotary_tables(positions, inv, cos, sin)
    results = []
    for fused in (False, True):
        q = torch.zeros(m, hq, dim, dtype=torch.bfloat16, device=dev())
        kc = torch.zeros(16 * n_req, hkv, page, dim, dtype=torch.bfloat16, device=dev()); vc = torch.zeros_like(kc)
        if fused:
            k.gemm_tcgen05_rope(hbf, w, dict(cos=cos, sin=sin, q_out=q, k_cache=kc, v_cache=vc, positions=positions, token_req=token_req,
                                             req_slot=req_slot, block_table=table, page_size=page, hq=hq, hkv=hkv, dim=dim))
            k.raise_if_kernel_gave_up()
        else:
            proj = torch.empty(m, w.shape[0], device=dev())
            k.gemm_library(hbf, w, proj)
            k.rope_store(proj, hq * dim, (hq + hkv) * dim, cos, sin, half, False, q, kc, vc, token_req, positions, req_slot, table,
                         page, hq, hkv, dim)
        results.append((q.float().cpu(), kc.float().cpu(), vc.float().cpu()))
    check_rotated_projection(results, plain_rotated_projection(hbf, w, positions, token_req, req_slot, table, page, 16 * n_req, hq, hkv,
                                                               dim, dim, False, theta))


def test_tensor_maps_of_one_launch_survive_an_eviction_between_them():
    """The library remembers tensor maps by (address, shape) and empties that cache when it is full.  A launch asks for
    two maps in a row (activations, then weights); with room for one entry only, the second request evicts the first
    while the launch still needs it.  The launch must use its own copies: the products stay right."""
    k = kernels()
    lib = k._tcgen05()
    lib.cisr_gemm_tcgen05_set_map_cache_limit(1)
    try:
        g = torch.Generator().manual_seed(5)
        for m, n, kk in ((200, 300, 128), (130, 64, 256), (200, 300, 128)):
            a = torch.randn(m, kk, generator=g).to(torch.bfloat16)
            w = torch.randn(n, kk, generator=g).to(torch.bfloat16)
            out = torch.full((m, n), float("nan"), device=dev())
            k.gemm_tcgen05(a.to(dev()), w.to(dev()), out)
            k.raise_if_kernel_gave_up()
            close(out, a.double() @ w.double().T, 2e-6 * kk ** 0.5 * 4, 1e-5, f"tcgen05 gemm {m}x{n}x{kk} with a one-entry map cache")
    finally:
        lib.cisr_gemm_tcgen05_set_map_cache_limit(4096)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,hq,hkv", [(64, 6, 2), (128, 8, 8)])
def test_decode_attention_of_a_request_does_not_depend_on_its_neighbours(dtype, d, hq, hkv):
    """Key ranges are cut at fixed absolute positions and empty ranges add exactly nothing, so a request's output is the
    same to the last bit alone, beside short requests, and beside a much longer one (which brings more ranges).  At head
    size 128 a warp's share of a range is two tiles: a launch of few CTAs requests both ahead, a launch of more CTAs
    than the device has SMs one after the other, and that must not show either."""
    k = kernels()
    from cisr_b200.parts.attention import DECODE_RANGE, decode_ranges
    page = 16
    lens = [700, 40, 3000, 257]
    i32 = lambda a: torch.as_tensor(np.asarray(list(a), dtype=np.int32), device=dev())
    g = torch.Generator().manual_seed(9)
    n_pages = sum(-(-n // page) for n in lens)
    kc = torch.randn(n_pages, hkv, page, d, generator=g).to(dtype).to(dev()); vc = torch.randn(n_pages, hkv, page, d, generator=g).to(dtype).to(dev())
    width = max(-(-n // page) for n in lens)
    table = np.full((len(lens), width), -1, dtype=np.int32)
    at = 0
    for r, n in enumerate(lens):
        need = -(-n // page)
        table[r, :need] = np.arange(at, at + need); at += need
    q_all = (2 * torch.randn(len(lens), hq, d, generator=g)).to(dtype).to(dev())

    def run(rows):
        n = len(rows)
        q = q_all[rows].contiguous()
        out = torch.full_like(q, float("nan"))
        n_splits = decode_ranges(max(lens[r] for r in rows))
        partial = torch.full((n, hq, n_splits, d), float("nan"), device=dev()); stats = torch.full((n, hq, n_splits, 2), float("nan"), device=dev())
        k.attn_decode(q, out, kc, vc, i32(rows), i32(table), i32(range(n)), n, i32(range(n)), i32([lens[r] for r in rows]), partial, stats,
                      hq, hkv, page, d ** -0.5, None, DECODE_RANGE, n_splits)
        return out

    alone = run([0])
    assert torch.isfinite(alone).all()
    pages0 = torch.as_tensor(table[0, :-(-lens[0] // page)].astype(np.int64), device=dev())
    keys = kc[pages0].permute(0, 2, 1, 3).reshape(-1, hkv, d)[:lens[0]].double().cpu()
    values = vc[pages0].permute(0, 2, 1, 3).reshape(-1, hkv, d)[:lens[0]].double().cpu()
    queries = torch.zeros(lens[0], hq, d, dtype=torch.float64); queries[-1] = q_all[0].double().cpu()
    close(alone[0], pl.causal_attention(queries, keys, values, None)[-1], *ATT_TOL[dtype], "decode attention of one request")
    assert torch.equal(run([1, 0])[1], alone[0])                 # beside a short request
    assert torch.equal(run([0, 2, 3, 1])[0], alone[0])           # beside a long one: twelve ranges instead of three
    assert torch.equal(run([3, 2])[0], run([3])[0])              # 257 keys: the second range holds one key


@pytest.mark.parametrize("d,hq,hkv,n_out", [(64, 9, 3, 576), (64, 32, 8, 200), (48, 5, 1, 240), (16, 2, 2, 64), (128, 4, 2, 96), (32, 16, 16, 130)])
@pytest.mark.parametrize("n_dec,longest", [(1, 1400), (8, 1400), (11, 1400), (16, 1400), (3, 5000), (8, 9000), (2, 20000)])
def test_merge_and_output_projection_in_one_launch(d, hq, hkv, n_out, n_dec, longest):
    """The cluster kernel that merges the key ranges and projects (merge_proj.cu) against the merge kernel followed by
    a float64 product: the merged rows must be the merge kernel's bfloat16 values exactly (a single differing bit in one
    of them would be a hundred times the bound), and the K-slices must add up to the whole product."""
    k = kernels()
    from cisr_b200.parts.attention import DECODE_RANGE, decode_ranges
    page = 16
    i32 = lambda a: torch.as_tensor(np.asarray(list(a), dtype=np.int32), device=dev())
    g = torch.Generator().manual_seed(d * hq + n_dec)
    # up to 16 key ranges: one batch of loads per element; up to 32: a second batch; beyond: the path through shared memory
    lens = [int(x) for x in torch.randint(1, longest + 100, (n_dec,), generator=g)]
    lens[0] = longest
    n_pages = sum(-(-n // page) for n in lens)
    kc = torch.randn(n_pages, hkv, page, d, generator=g).to(torch.bfloat16).to(dev())
    vc = torch.randn(n_pages, hkv, page, d, generator=g).to(torch.bfloat16).to(dev())
    table = np.full((n_dec, max(-(-n // page) for n in lens)), -1, dtype=np.int32)
    at = 0
    for r, n in enumerate(lens):
        need = -(-n // page)
        table[r, :need] = np.arange(at, at + need); at += need
    q = (2 * torch.randn(n_dec, hq, d, generator=g)).to(torch.bfloat16).to(dev())
    w = (torch.randn(n_out, hq * d, generator=g) / (hq * d) ** 0.5).to(torch.bfloat16).to(dev())
    rows = torch.randperm(n_dec, generator=g).tolist()            # request i's token sits in row rows[i] of the step
    q_rows = torch.empty_like(q); q_rows[rows] = q
    n_splits = decode_ranges(max(lens))
    if not k.merge_out_proj_ok(n_dec, hq, d, w):
        pytest.skip("not a shape for the cluster kernel")
    outs = {}
    for merge in (True, False):
        out = torch.full_like(q, float("nan"))
        partial = torch.full((n_dec, hq, n_splits, d), float("nan"), device=dev()); stats = torch.full((n_dec, hq, n_splits, 2), float("nan"), device=dev())
        k.attn_decode(q_rows, out, kc, vc, i32(range(n_dec)), i32(table), i32(range(n_dec)), n_dec, i32(rows), i32(lens), partial, stats,
                      hq, hkv, page, d ** -0.5, None, DECODE_RANGE, n_splits, merge=merge)
        outs[merge] = (out, partial, stats)
    merged = outs[True][0]                                          # bfloat16 rows [token row, hq, d] from the merge kernel
    assert torch.isnan(outs[False][0].float()).all()                # without the merge kernel `out` is not written
    projected = torch.full((n_dec, n_out), float("nan"), device=dev())
    k.merge_out_proj(outs[False][1], outs[False][2], n_splits, i32(range(n_dec)), i32(rows), n_dec, hq, d, w, projected)
    ref = merged.double().reshape(n_dec, hq * d) @ w.double().T
    close(projected, ref, 2e-6 * float(ref.abs().max()) + 1e-6, 1e-5, "merge + output projection")
    # the residual form: added to the rows of a stream that has more rows than the step has decoding requests' tokens
    stream = 10 * torch.randn(n_dec, n_out, generator=g)
    added = stream.clone().to(dev())
    k.merge_out_proj(outs[False][1], outs[False][2], n_splits, i32(range(n_dec)), i32(rows), n_dec, hq, d, w, added, accumulate=True)
    assert torch.equal(added.cpu(), stream + projected.cpu())

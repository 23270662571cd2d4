"""The decode attention entry point that allocates nothing (cisr_attn_decode_static).

Some users of the kernels cannot call cudaMalloc: plugin or callback code inside another runtime,
code held to a memory budget fixed at start-up, and bindings that have no tensor library to ask
for scratch.  For them the library keeps the scratch of the split decode attention in a static device
array.  This test calls the exported C symbol directly, as such a caller would, and checks its output
against the plain float64 attention (tests/plain_llama.py) and against the engine's own entry point
(caller-owned scratch) on calls in a row that share the array, then checks that an oversized call is
refused with a message.  It is collected last, so a run that stops at the first failure has already
run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HEAD_DIM = 64


def load(dtype):
    from cisr_b200.ops import build, kernels
    path = build.compile_library("attention_static_scratch.cu", {"HEAD_DIM": HEAD_DIM, "STORAGE_BF16": kernels.dtype_code(dtype)})
    lib = ctypes.CDLL(str(path))
    lib.cisr_attn_decode_static.restype = ctypes.c_int
    return lib


def make_case(seed, n_dec, hq, hkv, contexts, page_size, dtype):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-c // page_size) for c in contexts) + 2
    k_cache = torch.randn(n_pages, hkv, page_size, HEAD_DIM, generator=g).to(dtype).cuda()
    v_cache = torch.randn(n_pages, hkv, page_size, HEAD_DIM, generator=g).to(dtype).cuda()
    q = (2 * torch.randn(n_dec, hq, HEAD_DIM, generator=g)).to(dtype).cuda()
    width = max(-(-c // page_size) for c in contexts) + 1
    table = np.full((n_dec, width), -1, dtype=np.int32)
    perm = np.random.default_rng(seed).permutation(n_pages)
    at = 0
    for r, c in enumerate(contexts):
        need = -(-c // page_size)
        table[r, :need] = perm[at:at + need]
        at += need
    i32 = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32)).cuda()
    return dict(q=q, k=k_cache, v=v_cache, req_slot=i32(np.arange(n_dec)), table=i32(table), dec_req=i32(np.arange(n_dec)),
                q_start=i32(np.arange(n_dec)), ctx=i32(contexts), n_dec=n_dec, hq=hq, hkv=hkv, page_size=page_size, width=width)


def run_static(lib, c, split_size, n_splits, message=None):
    out = torch.full_like(c["q"], float("nan"))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    status = lib.cisr_attn_decode_static(
        p(c["q"]), p(out), p(c["k"]), p(c["v"]), p(c["req_slot"]), p(c["table"]), c["width"], p(c["dec_req"]), c["n_dec"],
        p(c["q_start"]), p(c["ctx"]), c["hq"], c["hkv"], c["page_size"], ctypes.c_float(HEAD_DIM ** -0.5), 0, split_size, n_splits,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), message, 0 if message is None else len(message))
    return status, out


def run_plain(c):
    """plain_llama.causal_attention in float64 on the stored (rounded) inputs: each request's keys and values gathered
    from its pages in order, its one query as the last row of a sequence whose earlier queries do not matter."""
    import plain_llama as pl
    q, kc, vc = c["q"].double().cpu(), c["k"].double().cpu(), c["v"].double().cpu()
    table, page = c["table"].cpu().numpy(), c["page_size"]
    out = torch.zeros_like(q)
    for r, n in enumerate(c["ctx"].cpu().tolist()):
        pages = [int(table[r, t // page]) for t in range(n)]
        keys = torch.stack([kc[pg, :, t % page] for t, pg in enumerate(pages)])        # [n, hkv, D]
        values = torch.stack([vc[pg, :, t % page] for t, pg in enumerate(pages)])
        queries = torch.zeros(n, c["hq"], HEAD_DIM, dtype=torch.float64)
        queries[-1] = q[r]
        out[r] = pl.causal_attention(queries, keys, values)[-1]
    return out


def run_engine(c, split_size, n_splits):
    from cisr_b200.ops import kernels
    out = torch.full_like(c["q"], float("nan"))
    partial = torch.empty(c["n_dec"], c["hq"], n_splits, HEAD_DIM, device="cuda")
    stats = torch.empty(c["n_dec"], c["hq"], n_splits, 2, device="cuda")
    kernels.attn_decode(c["q"], out, c["k"], c["v"], c["req_slot"], c["table"], c["dec_req"], c["n_dec"], c["q_start"], c["ctx"],
                        partial, stats, c["hq"], c["hkv"], c["page_size"], HEAD_DIM ** -0.5, None, split_size, n_splits)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_plain_and_the_engine_entry_point_on_calls_in_a_row(dtype):
    lib = load(dtype)
    first = make_case(1, n_dec=5, hq=9, hkv=3, contexts=[700, 64, 1, 333, 129], page_size=16, dtype=dtype)
    second = make_case(2, n_dec=3, hq=4, hkv=4, contexts=[90, 17, 250], page_size=8, dtype=dtype)
    for case, split_size in ((first, 64), (second, 128), (first, 256)):      # later calls find the earlier calls' leftovers
        n_splits = -(-max(case["ctx"].cpu().tolist()) // split_size)
        status, got = run_static(lib, case, split_size, n_splits)
        assert status == 0
        want = run_engine(case, split_size, n_splits)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # against float64 on the same stored inputs, at the bounds of the attention kernel tests (test_kernels_gpu.py)
        torch.testing.assert_close(got.double().cpu(), run_plain(case), atol=3e-6 if dtype == torch.float32 else 2e-2,
                                   rtol=1e-5 if dtype == torch.float32 else 2e-2)
        # and against the engine's entry point: float32 to rounding, bfloat16 to the last stored bit
        torch.testing.assert_close(got.float(), want.float(), atol=3e-6 if dtype == torch.float32 else 2e-2,
                                   rtol=1e-5 if dtype == torch.float32 else 2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = load(torch.float32)
    case = make_case(3, n_dec=4, hq=8, hkv=2, contexts=[100, 100, 100, 100], page_size=16, dtype=torch.float32)
    message = ctypes.create_string_buffer(400)
    n_splits = 20000                                     # 4 * 8 * 20000 * 66 floats is far beyond 8 MiB
    status, _ = run_static(lib, case, 64, n_splits, message)
    text = message.value.decode()
    assert status == -4 and "need" in text and "2097152" in text and "8388608" in text
    status, _ = run_static(lib, dict(case, hq=7), 64, 2, message)
    assert status == -2 and "multiple of hkv" in message.value.decode()
    status, got = run_static(lib, case, 64, 2)           # and it still works afterwards
    assert status == 0 and torch.isfinite(got).all()

"""The allocation-free decode attention entry point, called through its exported C symbol.

Some embedders of the kernels may not allocate device memory while they decode (a loop that must
not touch the allocator once running, a plug-in with a fixed budget).  For them the library offers
``mlr_attention_decode_static``: the same kernel as ``mlr_attention_decode``, with the scratch the
ordinary entry point takes from its caller kept in a fixed array inside the library.  This test
calls both symbols on the same inputs and requires identical output, twice in a row with
different inputs (the array keeps the first call's contents, which must not leak into the
second), and checks that a shape too large for the array is refused without a launch.
The file sorts last so that a run stopping at the first failure has run everything else first.
"""

import ctypes

import pytest
import torch

from mini_llm_runtime_b200.ops import build

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def pointer(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def make_case(seed, rows, heads, kv_heads, head_dim, page, longest):
    generator = torch.Generator().manual_seed(seed)
    contexts = torch.randint(1, longest, (rows,), generator=generator).tolist()
    contexts[0] = longest - 1
    pages_per_request = -(-longest // page)
    total_pages = rows * pages_per_request + 2
    order = torch.randperm(total_pages, generator=generator)[: rows * pages_per_request]
    table = order.reshape(rows, pages_per_request).to(torch.int32)
    k_pool = torch.randn(total_pages, kv_heads, page, head_dim, generator=generator).to(torch.bfloat16)
    v_pool = torch.randn(total_pages, kv_heads, page, head_dim, generator=generator).to(torch.bfloat16)
    q = torch.randn(rows, heads * head_dim, generator=generator).to(torch.bfloat16)
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=DEVICE)
    return {"q": q.to(DEVICE), "k": k_pool.to(DEVICE), "v": v_pool.to(DEVICE), "table": table.to(DEVICE),
            "decode_seg": ints(list(range(rows))), "q_start": ints(list(range(rows))), "pos0": ints(contexts),
            "contexts": contexts}


def call(lib, name, case, heads, kv_heads, head_dim, page, chunk, splits, extra=()):
    out = torch.zeros_like(case["q"])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # the ordinary entry point also takes the table row of each segment (null: row = segment)
    table_row = (ctypes.c_void_p(0),) if name == "mlr_attention_decode" else ()
    status = getattr(lib, name)(
        pointer(case["q"]), pointer(case["k"]), pointer(case["v"]), pointer(out), pointer(case["decode_seg"]),
        pointer(case["q_start"]), pointer(case["pos0"]), pointer(case["table"]), *table_row, case["table"].shape[1],
        case["q"].shape[0], heads, kv_heads, head_dim, page, 0, ctypes.c_float(head_dim ** -0.5), chunk, splits,
        *extra, stream)
    torch.cuda.synchronize()
    return status, out


def reference(case, heads, kv_heads, head_dim, page):
    """Plain float32 attention of each row over its own pages."""
    group = heads // kv_heads
    rows = case["q"].shape[0]
    out = torch.empty(rows, heads * head_dim)
    q = case["q"].float().cpu().view(rows, heads, head_dim)
    k_pool, v_pool, table = case["k"].float().cpu(), case["v"].float().cpu(), case["table"].cpu()
    for r, position in enumerate(case["contexts"]):
        keys = torch.arange(position + 1)
        pages, offsets = table[r, (keys // page).long()].long(), (keys % page).long()
        k = k_pool[pages, :, offsets].repeat_interleave(group, dim=1)
        v = v_pool[pages, :, offsets].repeat_interleave(group, dim=1)
        p = torch.softmax(torch.einsum("hd,khd->hk", q[r], k) * head_dim ** -0.5, dim=-1)
        out[r] = torch.einsum("hk,khd->hd", p, v).reshape(-1)
    return out


def test_allocation_free_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = build.load_library("attention_decode")
    lib.mlr_attention_decode_scratch.restype = ctypes.c_longlong
    lib.mlr_attention_decode_static_capacity.restype = ctypes.c_longlong
    heads, kv_heads, head_dim, page, chunk = 14, 2, 64, 16, 128
    for seed, rows, longest in ((1, 8, 1500), (2, 5, 700)):
        case = make_case(seed, rows, heads, kv_heads, head_dim, page, longest)
        splits = -(-longest // chunk)
        need = lib.mlr_attention_decode_scratch(rows, heads, head_dim, splits)
        assert need <= lib.mlr_attention_decode_static_capacity()
        scratch = torch.empty(need, dtype=torch.uint8, device=DEVICE)
        counters = torch.zeros(rows * kv_heads, dtype=torch.int32, device=DEVICE)
        status, ordinary = call(lib, "mlr_attention_decode", case, heads, kv_heads, head_dim, page, chunk, splits,
                                (pointer(scratch), pointer(counters)))
        assert status == 0
        before = torch.cuda.memory_allocated()
        status, static = call(lib, "mlr_attention_decode_static", case, heads, kv_heads, head_dim, page, chunk, splits)
        assert status == 0
        assert torch.equal(static, ordinary), "both entry points run the same kernel on the same inputs"
        assert torch.cuda.memory_allocated() - before < 65536     # only the test's own output tensor
        want = reference(case, heads, kv_heads, head_dim, page)
        error = (static.float().cpu() - want).norm(dim=-1) / want.norm(dim=-1)
        assert float(error.max()) <= 2e-2, "bfloat16 tolerance of the kernel tests"


def test_allocation_free_entry_point_refuses_what_its_array_cannot_hold():
    lib = build.load_library("attention_decode")
    heads, kv_heads, head_dim, page = 16, 2, 128, 16
    case = make_case(3, 64, heads, kv_heads, head_dim, page, 200)
    status, out = call(lib, "mlr_attention_decode_static", case, heads, kv_heads, head_dim, page, 32, 64)
    assert status == -4, "64 rows x 16 heads x 64 splits x 130 floats exceed the 4 MiB array"
    assert float(out.abs().sum()) == 0.0, "a refused call launches nothing"


def test_allocation_free_entry_point_checks_everything_before_it_enqueues_anything():
    """A chunk that is no multiple of 32 is refused by the kernel's own checks; the counters of the
    fixed array must not have been touched by then (the memset comes after every check)."""
    lib = build.load_library("attention_decode")
    heads, kv_heads, head_dim, page = 14, 2, 64, 16
    case = make_case(4, 4, heads, kv_heads, head_dim, page, 300)
    status, out = call(lib, "mlr_attention_decode_static", case, heads, kv_heads, head_dim, page, 48, 8)
    assert status == -2 and float(out.abs().sum()) == 0.0


def test_a_context_longer_than_the_grid_was_sized_for_is_still_right():
    """max_splits * chunk shorter than the longest context: the last CTA of a row walks on."""
    lib = build.load_library("attention_decode")
    heads, kv_heads, head_dim, page, chunk = 14, 2, 64, 16, 64
    case = make_case(5, 6, heads, kv_heads, head_dim, page, 900)
    status, out = call(lib, "mlr_attention_decode_static", case, heads, kv_heads, head_dim, page, chunk, 4)
    assert status == 0
    want = reference(case, heads, kv_heads, head_dim, page)
    error = (out.float().cpu() - want).norm(dim=-1) / want.norm(dim=-1)
    assert float(error.max()) <= 2e-2

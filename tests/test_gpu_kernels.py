"""Each CUDA kernel alone against a plain PyTorch float64 computation of the same operation, at sizes
other than the tiny models' (widths and vocabularies that are no power of two, head sizes in steps of
16, several group sizes, page sizes 1 to 32)."""
import math

import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tolerance(dtype):
    # relative to the largest magnitude of the expected tensor
    return 2e-6 if dtype == torch.float32 else 1e-2


def close(got, want, dtype, what, factor=1.0):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: {got.shape} != {want.shape}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    error = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert error <= tolerance(dtype) * factor, f"{what}: relative error {error:.3e}"


def rand(shape, dtype, seed, scale=1.0):
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=generator) * scale).to(dtype).to(DEVICE)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    from llmserver_b200 import ops
    table = rand((1000, 200), dtype, 1)
    ids = torch.tensor([0, 999, 5, 5, 321], dtype=torch.int32, device=DEVICE)
    out = ops.embedding(table, ids)
    assert out.dtype == torch.float32
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [80, 1000, 4096, 5120 + 48])
def test_add_rmsnorm(dtype, width):
    from llmserver_b200 import ops
    rows = 7
    residual = rand((rows, width), torch.float32, 2)
    delta = rand((rows, width), dtype, 3)
    weight = rand((width,), dtype, 4) + 1
    eps = 1e-5
    expected_residual = residual.double() + delta.double()
    expected = plain_model.rms_norm(expected_residual, weight.double(), eps)
    work = residual.clone()
    out = ops.add_rmsnorm(work, delta, weight, eps)
    close(work, expected_residual, torch.float32, "residual sum")
    close(out, expected, dtype, "add + norm")
    # without a delta the residual is only read
    work = residual.clone()
    out = ops.add_rmsnorm(work, None, weight, eps)
    assert torch.equal(work, residual)
    close(out, plain_model.rms_norm(residual.double(), weight.double(), eps), dtype, "norm")
    # selected rows: residual untouched, delta added on the fly
    picks = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEVICE)
    work = residual.clone()
    out = ops.add_rmsnorm(work, delta, weight, eps, rows=picks)
    assert torch.equal(work, residual)
    close(out, expected[picks.long()], dtype, "norm of selected rows")
    # a float32 weight beside bfloat16 activations
    if dtype == torch.bfloat16:
        out = ops.add_rmsnorm(residual.clone(), delta, weight.float(), eps, act_dtype=dtype)
        close(out, expected, dtype, "norm with a 32-bit weight")


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_and_silu_mul(dtype):
    from llmserver_b200 import ops
    x = rand((5, 176), dtype, 5)
    weight = rand((176,), dtype, 6) + 1
    close(ops.rmsnorm(x, weight, 1e-6), plain_model.rms_norm(x.double(), weight.double(), 1e-6), dtype, "rmsnorm")
    gate_up = rand((9, 2 * 1111), dtype, 7, 3.0)
    gate, up = gate_up.double()[:, :1111], gate_up.double()[:, 1111:]
    close(ops.silu_mul(gate_up), torch.nn.functional.silu(gate) * up, dtype, "silu_mul")
    # gate and up columns interleaved in groups of 64 (vector form) and of 5 (element-wise form)
    for inter, group in ((1152, 64), (1115, 5)):
        gate_up = rand((7, 2 * inter), dtype, 8, 3.0)
        blocks = gate_up.double().reshape(7, inter // group, 2, group)
        want = (torch.nn.functional.silu(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(7, inter)
        close(ops.silu_mul(gate_up, group=group), want, dtype, f"silu_mul in groups of {group}")


@pytest.mark.parametrize("rows,hidden,inter,split", [(1, 256, 128, 1), (8, 4096, 12288, 2), (37, 512, 1088, 3), (64, 1024, 2112, 4)])
def test_gate_up_product_with_the_gate_in_its_epilogue(rows, hidden, inter, split):
    """silu(x Wg^T) * (x Wu^T) from one kernel (gate and up rows interleaved in groups of 64 in the fused weight),
    against float64 and against the product followed by the activation kernel."""
    from llmserver_b200 import ops
    from llmserver_b200.ops import gemm_bf16
    dtype = torch.bfloat16
    x = rand((rows, hidden), dtype, 90)
    gate = (rand((inter, hidden), dtype, 91).float() * hidden ** -0.5 * 3).to(dtype)
    up = (rand((inter, hidden), dtype, 92).float() * hidden ** -0.5 * 3).to(dtype)
    weight = ops.interleave_gate_up(gate, up)
    assert torch.equal(weight[64:128], up[:64]) and torch.equal(weight[128:192], gate[64:128])
    gemm_bf16._choice[(gemm_bf16._row_bucket(rows), 2 * inter, hidden, gemm_bf16.OWN_KERNEL)] = split
    gemm_bf16._choice[(gemm_bf16._row_bucket(rows), 2 * inter, hidden, "gate-up-silu")] = split
    gemm_bf16._choice[(gemm_bf16._row_bucket(rows), 2 * inter, hidden, torch.bfloat16)] = split
    want = torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    launches = ops.launch_count()
    fused = ops.gate_up_silu(x, weight, ops.GATE_UP_GROUP)
    assert ops.launch_count() - launches == 1
    gemm_bf16.FUSE_GATE_UP_SILU = False
    try:
        apart = ops.gate_up_silu(x, weight, ops.GATE_UP_GROUP)
    finally:
        gemm_bf16.FUSE_GATE_UP_SILU = True
    torch.cuda.synchronize()
    gemm_bf16.check_errors()
    close(fused, want, dtype, "fused gate/up")
    close(apart, want, dtype, "gate/up product, then the activation kernel")


@pytest.mark.parametrize("shape", [(1, 7, 5), (33, 100, 77), (130, 257, 1000), (2, 509, 96), (64, 64, 16)])
def test_gemm_f32_is_true_32_bit(shape):
    from llmserver_b200 import ops
    m, n, k = shape
    x, w = rand((m, k), torch.float32, 8), rand((n, k), torch.float32, 9)
    out = ops.gemm_f32(x, w)
    close(out, x.double() @ w.double().T, torch.float32, f"gemm {shape}", factor=max(1.0, k / 200))
    # a row's result does not depend on the other rows of the call
    alone = ops.gemm_f32(x[m // 2:m // 2 + 1].contiguous(), w)
    assert torch.equal(alone[0], out[m // 2])


def test_linear_bf16():
    from llmserver_b200 import ops
    for m, n, k in [(1, 300, 128), (8, 509, 96), (70, 1000, 512), (300, 264, 200)]:
        x, w = rand((m, k), torch.bfloat16, 10), rand((n, k), torch.bfloat16, 11)
        want = x.double() @ w.double().T
        close(ops.linear(x, w), want, torch.bfloat16, f"linear bf16 {(m, n, k)}")
        out32 = ops.linear(x, w, out_dtype=torch.float32)
        assert out32.dtype == torch.float32
        close(out32, want, torch.bfloat16, f"linear bf16 -> f32 {(m, n, k)}")


@pytest.mark.parametrize("shape", [(1, 300, 128), (8, 509, 96), (64, 1000, 512), (17, 4096, 12288), (33, 200, 4096),
                                   (5, 128, 64), (3, 130, 72), (48, 6144, 4096), (16, 40000, 1024)])
def test_gemm_small_m_tcgen05(shape):
    """The tcgen05 / TMA product for few rows, called directly: ragged N and K, one K block, K split across a
    cluster (few tiles, long K), float32 and bfloat16 outputs."""
    from llmserver_b200.ops import gemm_bf16
    from llmserver_b200.ops.library import call, stream_handle
    m, n, k = shape
    assert gemm_bf16.small_m_supported(m, n, k)
    x, w = rand((m, k), torch.bfloat16, 12), rand((n, k), torch.bfloat16, 13, 0.05)
    want = x.double() @ w.double().T
    for out_dtype, split in ((torch.float32, 0), (torch.bfloat16, 0), (torch.float32, 3), (torch.bfloat16, 8)):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEVICE)
        call("llm_gemm_small_m", x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, n, int(out_dtype == torch.float32),
             split, *gemm_bf16.NO_SCALE, gemm_bf16.error_flag(DEVICE).data_ptr(), stream_handle())
        torch.cuda.synchronize()
        gemm_bf16.check_errors()
        close(out, want, out_dtype, f"small-M product {shape} -> {out_dtype}", factor=4.0 if out_dtype == torch.float32 else 1.0)


def paged(dense_k, dense_v, page_size, seed, dtype):
    """Scatters per-sequence dense K/V ([T, Hkv, D] each) into shuffled pages; returns pages, tables."""
    kv_heads, dim = dense_k[0].shape[1:]
    counts = [-(-k.shape[0] // page_size) for k in dense_k]
    total = sum(counts) + 3
    order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pages = torch.zeros((total, kv_heads, page_size, dim), dtype=dtype)
    v_pages = torch.zeros_like(k_pages)
    tables = torch.zeros((len(dense_k), max(counts)), dtype=torch.int32)
    for row, (k, v) in enumerate(zip(dense_k, dense_v)):
        for block in range(counts[row]):
            page = order.pop()
            tables[row, block] = page
            chunk = slice(block * page_size, min((block + 1) * page_size, k.shape[0]))
            k_pages[page, :, :chunk.stop - chunk.start] = k[chunk].transpose(0, 1)
            v_pages[page, :, :chunk.stop - chunk.start] = v[chunk].transpose(0, 1)
    return k_pages.to(DEVICE), v_pages.to(DEVICE), tables.to(DEVICE)


def plain_attention_rows(q, k, v, scale, window, first_query):
    """Rows first_query.. of plain causal attention; q [Tq, Hq, D] are the LAST Tq positions."""
    total = k.shape[0]
    full_q = torch.zeros((total,) + q.shape[1:], dtype=torch.float64)
    full_q[first_query:] = q
    return plain_model.causal_attention(full_q, k, v, scale, window)[first_query:]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,page_size,window", [
    (4, 2, 16, 4, None), (6, 1, 32, 8, None), (6, 3, 48, 16, 24), (8, 8, 64, 1, None), (5, 5, 80, 32, 7),
    (32, 8, 128, 16, None), (3, 1, 256, 16, 100)])
def test_attention_generic(dtype, heads, kv_heads, dim, page_size, window):
    """Mixed batch: a decode token of a long sequence, a prompt portion in the middle of another, a
    whole short prompt and a single first token."""
    from llmserver_b200 import ops
    contexts = [333, 150, 37, 1]      # tokens each sequence holds after the step
    q_lens = [1, 41, 37, 1]           # tokens of the step
    scale = dim ** -0.5
    dense_k = [rand((c, kv_heads, dim), dtype, 20 + i).cpu() for i, c in enumerate(contexts)]
    dense_v = [rand((c, kv_heads, dim), dtype, 30 + i).cpu() for i, c in enumerate(contexts)]
    k_pages, v_pages, tables = paged(dense_k, dense_v, page_size, 1, dtype)
    queries = [rand((n, heads, dim), dtype, 40 + i).cpu() for i, n in enumerate(q_lens)]
    q_stride = (heads + 2 * kv_heads) * dim
    packed = torch.zeros((sum(q_lens), q_stride), dtype=dtype)
    packed[:, :heads * dim] = torch.cat(queries).reshape(-1, heads * dim)
    positions = torch.cat([torch.arange(c - n, c) for c, n in zip(contexts, q_lens)]).to(torch.int32).to(DEVICE)
    seq_of_token = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(torch.int32).to(DEVICE)
    out = ops.attention_generic(packed.to(DEVICE), q_stride, k_pages, v_pages, tables, seq_of_token, positions,
                                heads, kv_heads, dim, scale, window or 0)
    want = torch.cat([plain_attention_rows(q.double(), k.double(), v.double(), scale, window, c - n)
                      for q, k, v, c, n in zip(queries, dense_k, dense_v, contexts, q_lens)])
    close(out, want, dtype, "attention")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_and_respects_the_window_edge(dtype):
    """One key among hundreds gets a score far above the rest, so the output must be its value: at
    position 3 of 700 (far away, first page), at a page's last slot, and at the two sides of a
    window's edge (the key at p - window + 1 is seen, the one at p - window is not)."""
    from llmserver_b200 import ops
    heads, kv_heads, dim, page_size = 2, 1, 32, 16
    context = 700
    direction = torch.zeros(dim)
    direction[5] = 1.0

    def run(hot_key, window):
        k = torch.randn((context, kv_heads, dim), generator=torch.Generator().manual_seed(1)) * 0.1
        v = torch.randn((context, kv_heads, dim), generator=torch.Generator().manual_seed(2))
        k[hot_key, 0] = direction * 40.0
        q = (direction * 40.0).repeat(1, heads, 1)
        k_pages, v_pages, tables = paged([k.to(dtype)], [v.to(dtype)], page_size, 3, dtype)
        q_stride = (heads + 2 * kv_heads) * dim
        packed = torch.zeros((1, q_stride), dtype=dtype)
        packed[:, :heads * dim] = q.reshape(1, -1).to(dtype)
        positions = torch.tensor([context - 1], dtype=torch.int32, device=DEVICE)
        seq = torch.zeros(1, dtype=torch.int32, device=DEVICE)
        out = ops.attention_generic(packed.to(DEVICE), q_stride, k_pages, v_pages, tables, seq, positions, heads,
                                    kv_heads, dim, 1.0, window)
        return out.float().cpu().view(heads, dim), v.to(dtype).float()

    for hot in (3, 15, 16, 687, 699):
        out, v = run(hot, 0)
        assert torch.allclose(out[0], v[hot, 0], atol=2e-2), f"key {hot} was not found"
    window = 100
    out, v = run(context - window, window)          # first key inside the window
    assert torch.allclose(out[1], v[context - window, 0], atol=2e-2)
    out, v = run(context - window - 1, window)      # last key outside the window
    assert not torch.allclose(out[1], v[context - window - 1, 0], atol=0.2)


@pytest.mark.parametrize("tokens,heads,kv_heads,hidden,qk_norm,weight_dtype", [
    (1, 8, 2, 256, True, torch.bfloat16), (5, 4, 4, 1024, True, torch.float32), (16, 32, 8, 4096, True, torch.bfloat16),
    (8, 6, 1, 512, False, torch.bfloat16), (41, 8, 2, 1024, True, torch.bfloat16), (64, 4, 1, 512, True, torch.float32)])
def test_qkv_projection_with_the_rotation_in_its_epilogue(tokens, heads, kv_heads, hidden, qk_norm, weight_dtype):
    """Heads of 128 and few tokens: the product kernel finishes each head itself (norm, rotation, cache write).  Against
    plain arithmetic in float64 and against the two separate kernels."""
    from llmserver_b200 import ops
    from llmserver_b200.ops import gemm_bf16
    dim, page_size, theta, eps, dtype = 128, 16, 1000000.0, 1e-6, torch.bfloat16
    width = (heads + 2 * kv_heads) * dim
    x = rand((tokens, hidden), dtype, 70)
    weight = (rand((width, hidden), dtype, 71).float() * hidden ** -0.5 * 4).to(dtype)
    q_weight = (rand((dim,), torch.float32, 72) + 1).to(weight_dtype) if qk_norm else None
    k_weight = (rand((dim,), torch.float32, 73) + 1).to(weight_dtype) if qk_norm else None
    positions = torch.tensor([(37 * i * i + 5) % 3000 for i in range(tokens)], dtype=torch.int32)
    seq_of_token = torch.arange(tokens, dtype=torch.int32)
    n_pages = tokens * (3000 // page_size + 1) + 1
    tables = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(9)).to(torch.int32).reshape(tokens, -1).contiguous()
    inv_freq = (1.0 / (theta ** (torch.arange(0, dim, 2).float() / dim))).to(DEVICE)
    results = {}
    # this package's kernel for the shape, with K divided into 1, 2 or 4 parts (a measurement may prefer the library's
    # product, which has no epilogue to fuse into)
    split = {1: 1, 5: 2, 8: 3, 16: 4, 41: 2, 64: 1}[tokens]
    gemm_bf16._choice[(gemm_bf16._row_bucket(tokens), width, hidden, gemm_bf16.OWN_KERNEL)] = split
    gemm_bf16._choice[(gemm_bf16._row_bucket(tokens), width, hidden, "qkv-rope")] = split
    for fused in (True, False):
        gemm_bf16.FUSE_QKV_ROPE = fused
        k_pages = torch.zeros((n_pages, kv_heads, page_size, dim), dtype=dtype, device=DEVICE)
        v_pages = torch.zeros_like(k_pages)
        flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
        launches = ops.launch_count()
        qkv = ops.qkv_projection(x, weight, q_weight, k_weight, inv_freq, positions.to(DEVICE), seq_of_token.to(DEVICE),
                                 tables.to(DEVICE), k_pages, v_pages, heads, kv_heads, dim, eps, True, flag)
        torch.cuda.synchronize()
        gemm_bf16.check_errors()
        assert flag.item() == 0
        results[fused] = (qkv[:, :heads * dim].float().cpu(), k_pages.float().cpu(), v_pages.float().cpu(), ops.launch_count() - launches)
    gemm_bf16.FUSE_QKV_ROPE = True
    assert results[True][3] < results[False][3], "the fused path was meant to launch fewer kernels"
    product = x.double().cpu() @ weight.double().cpu().T
    q = product[:, :heads * dim].view(tokens, heads, dim)
    k = product[:, heads * dim:(heads + kv_heads) * dim].view(tokens, kv_heads, dim)
    v = product[:, (heads + kv_heads) * dim:].view(tokens, kv_heads, dim)
    if qk_norm:
        q, k = plain_model.rms_norm(q, q_weight.double().cpu(), eps), plain_model.rms_norm(k, k_weight.double().cpu(), eps)
    cosine, sine = plain_model.rope_tables(positions, dim, theta, torch.float64)
    q, k = plain_model.apply_rope(q, cosine, sine), plain_model.apply_rope(k, cosine, sine)
    for fused in (True, False):
        got_q, got_k_pages, got_v_pages, _ = results[fused]
        close(got_q, q.reshape(tokens, -1), dtype, f"q (fused {fused})")
        got_k = torch.stack([got_k_pages[tables[t, p // page_size].item(), :, p % page_size] for t, p in enumerate(positions.tolist())])
        got_v = torch.stack([got_v_pages[tables[t, p // page_size].item(), :, p % page_size] for t, p in enumerate(positions.tolist())])
        close(got_k, k, dtype, f"cached k (fused {fused})")
        close(got_v, v, dtype, f"cached v (fused {fused})")
        written = (got_k_pages.abs().sum(dim=(1, 3)) > 0).sum().item()
        assert written == tokens, "slots other than the tokens' own were written"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,rotary,interleaved,qk_norm", [(48, 24, True, True), (128, 64, False, True), (128, 128, True, False),
                                                            (80, 2, False, True), (64, 0, False, True)])
def test_rotation_of_a_part_of_the_head_and_of_interleaved_pairs(dtype, dim, rotary, interleaved, qk_norm):
    """Only the first ``rotary`` elements of each head rotate, as halves or as neighbouring pairs; the rest is
    normalised and passes through.  rotary 0 with no frequencies: no position encoding at all."""
    from llmserver_b200 import ops
    heads, kv_heads, page_size, theta, eps = 3, 1, 8, 10000.0, 1e-6
    positions = torch.tensor([0, 1, 2, 3, 40, 41, 977], dtype=torch.int32)
    total, width = positions.numel(), (heads + 2 * kv_heads) * dim
    qkv = rand((total, width), dtype, 60)
    q_weight = rand((dim,), dtype, 61) + 1 if qk_norm else None
    k_weight = rand((dim,), dtype, 62) + 1 if qk_norm else None
    n_pages = 977 // page_size + 2
    tables = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, -1).contiguous()
    k_pages = torch.zeros((n_pages, kv_heads, page_size, dim), dtype=dtype, device=DEVICE)
    v_pages = torch.zeros_like(k_pages)
    flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    inv_freq = (1.0 / (theta ** (torch.arange(0, rotary, 2).float() / rotary))).to(DEVICE) if rotary else None
    work = qkv.clone()
    ops.qk_norm_rope_kv_write(work, q_weight, k_weight, inv_freq, positions.to(DEVICE), torch.zeros(total, dtype=torch.int32, device=DEVICE),
                              tables.to(DEVICE), k_pages, v_pages, heads, kv_heads, dim, eps, True, flag,
                              rotary_dim=rotary if rotary else None, interleaved=interleaved)
    assert flag.item() == 0
    source = qkv.double().cpu()
    q = source[:, :heads * dim].view(total, heads, dim)
    k = source[:, heads * dim:(heads + kv_heads) * dim].view(total, kv_heads, dim)
    if qk_norm:
        q, k = plain_model.rms_norm(q, q_weight.double().cpu(), eps), plain_model.rms_norm(k, k_weight.double().cpu(), eps)

    def rotated(x):
        if not rotary:
            return x
        angles = (positions.float().unsqueeze(-1) * inv_freq.cpu().view(1, -1)).double()
        cosine, sine = torch.cos(angles).unsqueeze(1), torch.sin(angles).unsqueeze(1)
        out = x.clone()
        first, second = (slice(0, rotary, 2), slice(1, rotary, 2)) if interleaved else (slice(0, rotary // 2), slice(rotary // 2, rotary))
        out[..., first] = x[..., first] * cosine - x[..., second] * sine
        out[..., second] = x[..., second] * cosine + x[..., first] * sine
        return out

    close(work[:, :heads * dim], rotated(q).reshape(total, -1), dtype, "rotated q")
    got_k = torch.stack([k_pages[tables[0, p // page_size].item(), :, p % page_size] for p in positions.tolist()])
    close(got_k, rotated(k), dtype, "cached k")
    with pytest.raises(ops.KernelError):
        ops.qk_norm_rope_kv_write(work, q_weight, k_weight, inv_freq, positions.to(DEVICE), torch.zeros(total, dtype=torch.int32, device=DEVICE),
                                  tables.to(DEVICE), k_pages, v_pages, heads, kv_heads, dim, eps, True, flag, rotary_dim=dim + 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,page_size,qk_norm", [(4, 2, 16, 4, True), (6, 1, 48, 16, True),
                                                                  (8, 8, 128, 16, False), (5, 5, 80, 3, True)])
def test_qk_norm_rope_kv_write(dtype, heads, kv_heads, dim, page_size, qk_norm):
    from llmserver_b200 import ops
    starts, counts = [130, 0, 77], [1, 19, 6]
    theta, eps = 50000.0, 1e-5
    total = sum(counts)
    width = (heads + 2 * kv_heads) * dim
    qkv = rand((total, width), dtype, 50)
    q_weight = rand((dim,), dtype, 51) + 1 if qk_norm else None
    k_weight = rand((dim,), dtype, 52) + 1 if qk_norm else None
    positions = torch.cat([torch.arange(s, s + c) for s, c in zip(starts, counts)])
    seq_of_token = torch.cat([torch.full((c,), i) for i, c in enumerate(counts)])
    pages_per_seq = [-(-(s + c) // page_size) for s, c in zip(starts, counts)]
    n_pages = sum(pages_per_seq) + 2
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(4)).tolist()
    tables = torch.zeros((3, max(pages_per_seq)), dtype=torch.int32)
    for row, count in enumerate(pages_per_seq):
        for block in range(count):
            tables[row, block] = order.pop()
    k_pages = torch.zeros((n_pages, kv_heads, page_size, dim), dtype=dtype, device=DEVICE)
    v_pages = torch.zeros_like(k_pages)
    flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    inv_freq = (1.0 / (theta ** (torch.arange(0, dim, 2).float() / dim))).to(DEVICE)
    work = qkv.clone()
    ops.qk_norm_rope_kv_write(work, q_weight, k_weight, inv_freq, positions.to(torch.int32).to(DEVICE),
                              seq_of_token.to(torch.int32).to(DEVICE), tables.to(DEVICE), k_pages, v_pages, heads,
                              kv_heads, dim, eps, True, flag)
    assert flag.item() == 0
    source = qkv.double().cpu()
    q = source[:, :heads * dim].view(total, heads, dim)
    k = source[:, heads * dim:(heads + kv_heads) * dim].view(total, kv_heads, dim)
    v = source[:, (heads + kv_heads) * dim:].view(total, kv_heads, dim)
    if qk_norm:
        q = plain_model.rms_norm(q, q_weight.double().cpu(), eps)
        k = plain_model.rms_norm(k, k_weight.double().cpu(), eps)
    cosine, sine = plain_model.rope_tables(positions, dim, theta, torch.float64)
    q, k = plain_model.apply_rope(q, cosine, sine), plain_model.apply_rope(k, cosine, sine)
    close(work[:, :heads * dim], q.reshape(total, -1), dtype, "rotated q")
    got_k = torch.stack([k_pages[tables[s, p // page_size].item(), :, p % page_size]
                         for s, p in zip(seq_of_token.tolist(), positions.tolist())])
    got_v = torch.stack([v_pages[tables[s, p // page_size].item(), :, p % page_size]
                         for s, p in zip(seq_of_token.tolist(), positions.tolist())])
    close(got_k, k, dtype, "cached k")
    assert torch.equal(got_v.cpu(), qkv[:, (heads + kv_heads) * dim:].view(total, kv_heads, dim).cpu()), "cached v is a copy"
    written = (k_pages.float().abs().sum(dim=(1, 3)) > 0).sum().item()
    assert written == total, "slots other than the tokens' own were written"
    # an entry that reads another entry's cache rotates q and leaves the pages alone
    before = k_pages.clone()
    again = qkv.clone()
    ops.qk_norm_rope_kv_write(again, q_weight, k_weight, inv_freq, positions.to(torch.int32).to(DEVICE),
                              seq_of_token.to(torch.int32).to(DEVICE), tables.to(DEVICE), k_pages, v_pages, heads,
                              kv_heads, dim, eps, False, flag)
    assert torch.equal(before, k_pages) and torch.equal(again[:, :heads * dim], work[:, :heads * dim])


def test_sampling_greedy_and_temperature():
    from llmserver_b200 import ops
    vocab = 5003
    logits = rand((6, vocab), torch.float32, 60, 2.0)
    logits[2, 77] = logits[2, 4000] = logits[2].max() + 1.0   # a tie: the lower index wins
    tokens = ops.sample(logits).cpu()
    assert tokens.tolist() == torch.argmax(logits.cpu(), dim=-1).tolist()
    assert tokens[2].item() == 77
    temperatures = torch.tensor([0.8, 0.0, 1.5, 0.8, 0.3, 1.0], dtype=torch.float32, device=DEVICE)
    seeds = torch.tensor([1, 2, 3, 1, 2 ** 40 + 5, 7], dtype=torch.int64, device=DEVICE)
    steps = torch.tensor([0, 0, 5, 1, 9, 1000], dtype=torch.int32, device=DEVICE)
    drawn = ops.sample(logits, temperatures, seeds, steps).cpu().tolist()
    again = ops.sample(logits[[3, 0]].contiguous(), temperatures[[3, 0]].contiguous(), seeds[[3, 0]].contiguous(),
                       steps[[3, 0]].contiguous()).cpu().tolist()
    assert again == [drawn[3], drawn[0]], "a row's draw depends on its place in the batch"
    host = logits.cpu()
    for row, token in enumerate(drawn):
        if temperatures[row].item() == 0.0:
            assert token == int(torch.argmax(host[row]))
            continue
        scores = plain_model.gumbel_scores(host[row], temperatures[row].item(), int(seeds[row]), int(steps[row]))
        assert scores[token] >= scores.max() - 1e-4, f"row {row}: token {token} is not the Gumbel-max choice"
    # the noise depends on the step: the same row drawn at 64 different steps does not give one token 64 times
    many = torch.arange(64, dtype=torch.int32, device=DEVICE)
    row = 1 if temperatures[1].item() > 0 else int((temperatures > 0).nonzero()[0])
    tokens = ops.sample(logits[row:row + 1].expand(64, -1).contiguous(), temperatures[row:row + 1].expand(64).contiguous(),
                        seeds[row:row + 1].expand(64).contiguous(), many).cpu().tolist()
    assert len(set(tokens)) > 1, "the draw does not depend on the step"


def test_sampling_over_a_large_vocabulary():
    """Vocabularies from 16384 up are scanned by several blocks per row and merged by a second kernel."""
    from llmserver_b200 import ops
    vocab = 151936
    logits = rand((3, vocab), torch.float32, 61, 2.0)
    logits[1, 150000] = logits[1, 9000] = logits[1].max() + 1.0     # a tie across slices: the lower index wins
    assert ops.sample(logits).cpu().tolist() == torch.argmax(logits.cpu(), dim=-1).tolist()
    assert ops.sample(logits)[1].item() == 9000
    temperatures = torch.tensor([0.7, 1.0, 0.0], dtype=torch.float32, device=DEVICE)
    seeds = torch.tensor([5, 6, 7], dtype=torch.int64, device=DEVICE)
    steps = torch.tensor([3, 4, 5], dtype=torch.int32, device=DEVICE)
    drawn = ops.sample(logits, temperatures, seeds, steps).cpu().tolist()
    host = logits.cpu()
    for row in (0, 1):
        scores = plain_model.gumbel_scores(host[row], temperatures[row].item(), int(seeds[row]), int(steps[row]))
        assert scores[drawn[row]] >= scores.max() - 1e-4
    assert drawn[2] == int(torch.argmax(host[2]))


def test_sampling_follows_the_distribution():
    from llmserver_b200 import ops
    probabilities = torch.tensor([0.5, 0.25, 0.125, 0.125])
    draws = 4000
    logits = probabilities.log().repeat(draws, 1).to(DEVICE).contiguous()
    temperatures = torch.ones(draws, device=DEVICE)
    seeds = torch.full((draws,), 12345, dtype=torch.int64, device=DEVICE)
    steps = torch.arange(draws, dtype=torch.int32, device=DEVICE)
    tokens = ops.sample(logits, temperatures, seeds, steps).cpu()
    observed = torch.bincount(tokens.long(), minlength=4).double() / draws
    assert (observed - probabilities.double()).abs().max() < 4 * math.sqrt(0.25 / draws)


class FakeBatch:
    """The fields of a step batch that the attention wrappers read."""

    def __init__(self, contexts, q_lens):
        self.q_lens, self.context_lens = list(q_lens), list(contexts)
        self.n_seqs, self.n_tokens = len(q_lens), sum(q_lens)
        self.max_context = max(contexts)
        starts = [0]
        for n in q_lens:
            starts.append(starts[-1] + n)
        self.q_start = torch.tensor(starts, dtype=torch.int32, device=DEVICE)
        self.context_len = torch.tensor(contexts, dtype=torch.int32, device=DEVICE)
        self.positions = torch.cat([torch.arange(c - n, c) for c, n in zip(contexts, q_lens)]).to(torch.int32).to(DEVICE)
        self.seq_of_token = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(torch.int32).to(DEVICE)
        self.scratch = {}


@pytest.mark.parametrize("heads,kv_heads,dim,page_size,window", [
    (32, 8, 128, 16, None), (6, 1, 64, 8, None), (8, 8, 128, 1, None), (16, 1, 64, 16, 100), (12, 4, 128, 32, 300),
    (5, 5, 64, 3, None)])
@pytest.mark.parametrize("shape", ["decode", "portions", "mixed"])
def test_attention_tensor_core_kernels(heads, kv_heads, dim, page_size, window, shape):
    """The bfloat16 tensor-core kernels (prompt portions, split-KV decode, both in one mixed batch)
    against plain attention: contexts long enough for several splits, portions that start in the middle
    of a page and of a 64-key tile, a single first token, rows that are no multiple of the tile."""
    from llmserver_b200 import ops
    from llmserver_b200.ops import attention_bf16
    assert attention_bf16.supported(dim, heads, kv_heads)
    dtype = torch.bfloat16
    if shape == "decode":
        contexts, q_lens = [1500, 257, 64, 1, 700], [1, 1, 1, 1, 1]
    elif shape == "portions":
        contexts, q_lens = [333, 150, 37, 900], [41, 150, 2, 130]
    else:
        contexts, q_lens = [1100, 333, 1, 77, 513], [1, 70, 1, 77, 1]
    scale = dim ** -0.5
    dense_k = [rand((c, kv_heads, dim), dtype, 120 + i).cpu() for i, c in enumerate(contexts)]
    dense_v = [rand((c, kv_heads, dim), dtype, 130 + i).cpu() for i, c in enumerate(contexts)]
    k_pages, v_pages, tables = paged(dense_k, dense_v, page_size, 7, dtype)
    queries = [rand((n, heads, dim), dtype, 140 + i).cpu() for i, n in enumerate(q_lens)]
    q_stride = (heads + 2 * kv_heads) * dim
    packed = torch.zeros((sum(q_lens), q_stride), dtype=dtype)
    packed[:, :heads * dim] = torch.cat(queries).reshape(-1, heads * dim)
    batch = FakeBatch(contexts, q_lens)
    out = attention_bf16.try_attention(packed.to(DEVICE), q_stride, batch, tables, k_pages, v_pages, heads, kv_heads,
                                       dim, scale, window or 0)
    assert out is not None
    want = torch.cat([plain_attention_rows(q.double(), k.double(), v.double(), scale, window, c - n)
                      for q, k, v, c, n in zip(queries, dense_k, dense_v, contexts, q_lens)])
    close(out, want, dtype, f"tensor-core attention ({shape})")
    # and the generic kernel agrees on the same inputs
    generic = ops.attention_generic(packed.to(DEVICE), q_stride, k_pages, v_pages, tables, batch.seq_of_token,
                                    batch.positions, heads, kv_heads, dim, scale, window or 0)
    close(generic, want, dtype, "generic attention on the same batch")


@pytest.mark.parametrize("kernel,pairing", [("tcgen05", None), ("tcgen05-128", True), ("tcgen05-256", False), ("tcgen05-256", True), ("mma", None)])
def test_tensor_core_attention_finds_a_far_key_and_respects_the_window_edge(kernel, pairing):
    """One key among 1300 is made to stand out for the last query (score 1600 against about 0): every kernel that
    can run a decode token or a portion of 40 has to return that key's value, wherever the key lies (first tile, a
    tile's edge, just inside or just outside the window).  The jump of the maximum also sends the kernels through
    their rescaling paths."""
    from llmserver_b200.ops import attention_bf16
    heads, kv_heads, dim, page_size, context = 4, 1, 128, 16, 1300
    dtype = torch.bfloat16
    direction = torch.zeros(dim)
    direction[9] = 1.0
    attention_bf16.PREFILL_KERNEL, attention_bf16.FORCE_PAIRING = kernel, pairing
    try:
        for q_len in (1, 40) if kernel == "tcgen05" else (40,):
            for hot, window, found in ((3, 0, True), (255, 0, True), (256, 0, True), (1299 - 40, 0, True),
                                       (context - 200, 200, True), (context - 201, 200, False)):
                k = torch.randn((context, kv_heads, dim), generator=torch.Generator().manual_seed(1)) * 0.1
                v = torch.randn((context, kv_heads, dim), generator=torch.Generator().manual_seed(2))
                k[hot, 0] = direction * 40.0
                q = torch.zeros((q_len, heads, dim))
                q[-1] = direction * 40.0       # the last query looks for the hot key
                k_pages, v_pages, tables = paged([k.to(dtype)], [v.to(dtype)], page_size, 3, dtype)
                q_stride = (heads + 2 * kv_heads) * dim
                packed = torch.zeros((q_len, q_stride), dtype=dtype)
                packed[:, :heads * dim] = q.reshape(q_len, -1).to(dtype)
                batch = FakeBatch([context], [q_len])
                out = attention_bf16.try_attention(packed.to(DEVICE), q_stride, batch, tables, k_pages, v_pages, heads,
                                                   kv_heads, dim, 1.0, window)
                last = out[-1].float().cpu().view(heads, dim)[2]
                target = v.to(dtype).float()[hot, 0]
                assert torch.allclose(last, target, atol=3e-2) == found, f"q_len {q_len}, hot key {hot}, window {window}"
    finally:
        attention_bf16.PREFILL_KERNEL, attention_bf16.FORCE_PAIRING = "tcgen05", None


@pytest.mark.parametrize("heads,kv_heads,page_size,window", [(32, 8, 16, None), (4, 4, 8, None), (16, 1, 32, 100),
                                                             (8, 4, 64, None), (8, 1, 16, 300), (2, 1, 16, None),
                                                             (40, 8, 16, None), (3, 1, 16, 100), (12, 2, 32, None), (7, 1, 8, None)])
def test_attention_prefill_tcgen05(heads, kv_heads, page_size, window):
    """The two tcgen05 / tensor-memory kernels for prompt portions (128 and 256 rows per block; head_dim 128, groups
    of 1 to 16 heads, whole pages per tile): portions that start in the middle of a page and of a tile, more than
    one row tile, a whole prompt, a portion of two tokens, beside single tokens that go to the decode kernel; groups
    of 5, 3, 6 and 7 heads, which leave the last rows of a tile idle."""
    from llmserver_b200.ops import attention_bf16
    dim, dtype = 128, torch.bfloat16
    assert attention_bf16.prefill_tcgen05_supported(dim, heads, kv_heads, page_size)
    contexts, q_lens = [1100, 333, 1, 77, 513, 700], [1, 70, 1, 77, 2, 300]
    scale = dim ** -0.5
    dense_k = [rand((c, kv_heads, dim), dtype, 220 + i).cpu() for i, c in enumerate(contexts)]
    dense_v = [rand((c, kv_heads, dim), dtype, 230 + i).cpu() for i, c in enumerate(contexts)]
    k_pages, v_pages, tables = paged(dense_k, dense_v, page_size, 9, dtype)
    queries = [rand((n, heads, dim), dtype, 240 + i).cpu() for i, n in enumerate(q_lens)]
    q_stride = (heads + 2 * kv_heads) * dim
    packed = torch.zeros((sum(q_lens), q_stride), dtype=dtype)
    packed[:, :heads * dim] = torch.cat(queries).reshape(-1, heads * dim)
    want = torch.cat([plain_attention_rows(q.double(), k.double(), v.double(), scale, window, c - n)
                      for q, k, v, c, n in zip(queries, dense_k, dense_v, contexts, q_lens)])
    results = {}
    for kernel, pairing in (("tcgen05-128", False), ("tcgen05-128", True), ("tcgen05-256", False), ("tcgen05-256", True), ("mma", None)):
        attention_bf16.PREFILL_KERNEL, attention_bf16.FORCE_PAIRING = kernel, pairing
        try:
            out = attention_bf16.try_attention(packed.to(DEVICE), q_stride, FakeBatch(contexts, q_lens), tables, k_pages, v_pages,
                                               heads, kv_heads, dim, scale, window or 0)
        finally:
            attention_bf16.PREFILL_KERNEL, attention_bf16.FORCE_PAIRING = "tcgen05", None
        torch.cuda.synchronize()
        from llmserver_b200.ops import gemm_bf16
        gemm_bf16.check_errors()
        close(out, want, dtype, f"prompt attention ({kernel}, tiles {'paired' if pairing else 'one by one'})")
        if pairing is not False:
            results[kernel] = out
    close(results["tcgen05-128"], results["mma"].double().cpu(), dtype, "the 128-row kernel against the mma.sync kernel")
    close(results["tcgen05-256"], results["mma"].double().cpu(), dtype, "the 256-row kernel against the mma.sync kernel")


def test_float32_logits_are_32_bit_sums_whatever_the_number_of_rows():
    """The output head's product: float32 results come from 32-bit accumulators for 64 rows, for 65 (two launches of
    this package's kernel) and for a shape the kernel does not take (the library's product with a 32-bit result), never
    from a bfloat16 product widened afterwards.  A row's logits do not depend on how many rows share the step beyond the
    order of a 32-bit sum."""
    from llmserver_b200 import ops
    hidden, vocab = 512, 5003
    x = rand((130, hidden), torch.bfloat16, 31)
    head = rand((vocab, hidden), torch.bfloat16, 32, 0.05)
    want = x.double() @ head.double().T
    scale = want.abs().max().item()
    by_rows = {}
    for rows in (1, 64, 65, 130):
        got = ops.linear(x[:rows].contiguous(), head, out_dtype=torch.float32)
        assert got.dtype == torch.float32
        assert (got.bfloat16().float() != got).float().mean().item() > 0.9, f"{rows} rows: the logits look rounded to bfloat16"
        assert (got.double() - want[:rows]).abs().max().item() <= 2e-5 * scale, f"{rows} rows: not a 32-bit sum"
        by_rows[rows] = got
    assert (by_rows[65][:64] - by_rows[64]).abs().max().item() <= 2e-6 * scale
    assert (by_rows[130][:1] - by_rows[1]).abs().max().item() <= 2e-6 * scale
    odd = rand((70, 100), torch.bfloat16, 33)            # an inner size that is no multiple of 8: the library's product
    odd_head = rand((300, 100), torch.bfloat16, 34)
    got = ops.linear(odd, odd_head, out_dtype=torch.float32)
    assert (got.double() - odd.double() @ odd_head.double().T).abs().max().item() <= 2e-5 * got.abs().max().item()
    assert (got.bfloat16().float() != got).float().mean().item() > 0.9


def test_the_microbenchmarks_run(capsys):
    """The workloads the profiler is pointed at, at small sizes: each must run and print its JSON line."""
    import json
    from llmserver_b200.cli import microbench
    for arguments in (["gemm", "--rows", "8", "--out-features", "1024", "--in-features", "512"],
                      ["attention-decode", "--batch", "3", "--context", "300"],
                      ["attention-prefill", "--tokens", "300"],
                      ["attention-prefill", "--tokens", "128", "--context", "700", "--shuffle-pages"]):
        assert microbench.main(arguments) == 0
        report = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert report["workload"] == arguments[0] and report.get("us", report.get("tcgen05_us", 0)) > 0


@pytest.mark.parametrize("rows,cols,inner,split,weight_dtype,with_norm", [
    (1, 4096, 12288, 0, torch.bfloat16, True), (8, 4096, 4096, 4, torch.bfloat16, True), (16, 200, 136, 1, torch.float32, True),
    (5, 1000, 512, 2, torch.bfloat16, True), (3, 328, 264, 0, torch.bfloat16, False),
    (7, 326, 264, 3, torch.bfloat16, True), (2, 130, 72, 1, torch.float32, True)])      # widths that are no multiple of four
def test_product_added_to_the_stream_in_its_epilogue(rows, cols, inner, split, weight_dtype, with_norm):
    """residual += x W^T inside the product kernel, with the next norm's input prepared: the stream times the norm's
    weight and, in parts, the rows' sums of squares."""
    from llmserver_b200 import ops
    from llmserver_b200.ops import gemm_bf16
    x, w = rand((rows, inner), torch.bfloat16, 31), rand((cols, inner), torch.bfloat16, 32, 0.05)
    residual = rand((rows, cols), torch.float32, 33)
    norm_weight = (rand((cols,), weight_dtype, 34) + 1) if with_norm else None
    want = residual.double() + x.double() @ w.double().T
    if split:
        gemm_bf16._choice[(gemm_bf16._row_bucket(rows), cols, inner, gemm_bf16.OWN_KERNEL)] = split
    sink = ops.StreamSink(residual, norm_weight, 1e-5)
    assert ops.linear(x, w, sink=sink) is None and sink.added
    torch.cuda.synchronize()
    gemm_bf16.check_errors()
    close(residual, want, torch.float32, "stream after the product", factor=8.0)      # 32-bit sums of bfloat16 products
    if not with_norm:
        assert sink.scaled is None
        return
    scaled = sink.scaled
    assert scaled.x.dtype == torch.bfloat16 and scaled.eps == 1e-5
    close(scaled.x, residual.double() * norm_weight.double(), torch.bfloat16, "stream times the norm's weight")
    squares = scaled.parts.double().sum(0)[:rows]
    close(squares, (residual.double() ** 2).sum(1), torch.float32, "sums of squares", factor=4.0)


@pytest.mark.parametrize("rows,width,cols", [(1, 4096, 6144), (8, 4096, 1000), (16, 264, 328), (5, 5120, 512)])
def test_products_divide_unscaled_rows_by_their_root_mean_square(rows, width, cols):
    """A product given the stream times the norm's weight and the sums of squares equals the product of the
    normalised rows: from the stand-alone norm kernel and from a product's stream epilogue, in one part or many."""
    from llmserver_b200 import ops
    from llmserver_b200.ops import gemm_bf16
    eps = 1e-6
    residual = rand((rows, width), torch.float32, 41, 3.0)
    norm_weight = rand((width,), torch.bfloat16, 42) + 1
    w = rand((cols, width), torch.bfloat16, 43, 0.05)
    normed = plain_model.rms_norm(residual.double(), norm_weight.double(), eps)
    want = normed @ w.double().T
    unscaled = ops.add_rmsnorm(residual.clone(), None, norm_weight, eps, act_dtype=torch.bfloat16, unscaled=True)
    assert isinstance(unscaled, ops.RowScaled) and unscaled.parts.shape[0] == 1
    for out_dtype in (torch.bfloat16, torch.float32):
        got = ops.linear(unscaled, w, out_dtype=out_dtype)
        torch.cuda.synchronize()
        gemm_bf16.check_errors()
        close(got, want, torch.bfloat16, f"product of unscaled rows -> {out_dtype}")
    # the same rows prepared by a product's epilogue (many parts): stream = 0 + previous product
    previous_x, previous_w = rand((rows, 136), torch.bfloat16, 44), rand((width, 136), torch.bfloat16, 45, 0.3)
    stream = torch.zeros((rows, width), dtype=torch.float32, device=DEVICE)
    sink = ops.StreamSink(stream, norm_weight, eps)
    assert ops.linear(previous_x, previous_w, sink=sink) is None
    assert sink.scaled.parts.shape[0] == -(-width // 128)
    got = ops.linear(sink.scaled, w)
    torch.cuda.synchronize()
    gemm_bf16.check_errors()
    want = plain_model.rms_norm(stream.double(), norm_weight.double(), eps) @ w.double().T
    close(got, want, torch.bfloat16, "product of rows prepared by a product")


def test_gate_up_and_qkv_products_take_unscaled_rows():
    from llmserver_b200 import ops
    from llmserver_b200.ops import gemm_bf16
    rows, hidden, inter, eps = 6, 1024, 640, 1e-6
    residual = rand((rows, hidden), torch.float32, 51, 2.0)
    norm_weight = rand((hidden,), torch.bfloat16, 52) + 1
    gate, up = rand((inter, hidden), torch.bfloat16, 53, 0.05), rand((inter, hidden), torch.bfloat16, 54, 0.05)
    normed = ops.add_rmsnorm(residual.clone(), None, norm_weight, eps, act_dtype=torch.bfloat16)
    unscaled = ops.add_rmsnorm(residual.clone(), None, norm_weight, eps, act_dtype=torch.bfloat16, unscaled=True)
    fused_weight = ops.interleave_gate_up(gate, up)
    before = ops.launch_count()
    got = ops.gate_up_silu(unscaled, fused_weight, ops.GATE_UP_GROUP)
    assert ops.launch_count() - before == 1 or gemm_bf16.tunings() > 0
    want = ops.gate_up_silu(normed, fused_weight, ops.GATE_UP_GROUP)
    torch.cuda.synchronize()
    gemm_bf16.check_errors()
    close(got, want.double(), torch.bfloat16, "gate/up product of unscaled rows")
    # q/k/v projection with the rotation in its epilogue
    heads, kv_heads, dim, page_size = 4, 2, 128, 16
    qkv_weight = rand(((heads + 2 * kv_heads) * dim, hidden), torch.bfloat16, 55, 0.05)
    q_norm, k_norm = rand((dim,), torch.bfloat16, 56) + 1, rand((dim,), torch.bfloat16, 57) + 1
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))).to(DEVICE)
    positions = torch.arange(3, 3 + rows, dtype=torch.int32, device=DEVICE)
    seq_of_token = torch.zeros(rows, dtype=torch.int32, device=DEVICE)
    tables = torch.tensor([[2, 1, 0, 3]], dtype=torch.int32, device=DEVICE)
    flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    results = []
    for x in (unscaled, normed):
        k_pages = torch.zeros((4, kv_heads, page_size, dim), dtype=torch.bfloat16, device=DEVICE)
        v_pages = torch.zeros_like(k_pages)
        qkv = ops.qkv_projection(x, qkv_weight, q_norm, k_norm, inv_freq, positions, seq_of_token, tables, k_pages, v_pages,
                                 heads, kv_heads, dim, eps, True, flag)
        results.append((qkv[:, :heads * dim].clone(), k_pages, v_pages))
    torch.cuda.synchronize()
    gemm_bf16.check_errors()
    assert flag.item() == 0
    for got, want, what in zip(results[0], results[1], ("q", "k pages", "v pages")):
        close(got, want.double(), torch.bfloat16, f"q/k/v projection of unscaled rows: {what}", factor=2.0)


@pytest.mark.parametrize("contexts,heads,kv_heads,splits", [([3000], 8, 2, 16), ([2900, 1300], 12, 4, 16), ([2000], 8, 2, 8), ([3000] * 5, 8, 2, 8)])
def test_decode_attention_in_clusters_of_sixteen(contexts, heads, kv_heads, splits):
    """With so few (sequence, kv head) pairs that sixteen blocks each still have an SM of their own, long contexts are
    split sixteen ways and merged inside a cluster of sixteen blocks; with more pairs or shorter contexts up to eight."""
    from llmserver_b200.ops import attention_bf16
    dim, page_size, dtype = 128, 16, torch.bfloat16
    q_lens = [1] * len(contexts)
    scale = dim ** -0.5
    dense_k = [rand((c, kv_heads, dim), dtype, 220 + i).cpu() for i, c in enumerate(contexts)]
    dense_v = [rand((c, kv_heads, dim), dtype, 230 + i).cpu() for i, c in enumerate(contexts)]
    # one far key per sequence that a lost split would lose: it takes most of the weight of head 0
    queries = [rand((1, heads, dim), dtype, 240 + i).cpu() for i in range(len(contexts))]
    for i, c in enumerate(contexts):
        far = (c * (i + 3)) // 9
        dense_k[i][far, 0] = queries[i][0, 0] * 3.0
    k_pages, v_pages, tables = paged(dense_k, dense_v, page_size, 5, dtype)
    q_stride = (heads + 2 * kv_heads) * dim
    packed = torch.zeros((len(contexts), q_stride), dtype=dtype)
    packed[:, :heads * dim] = torch.cat(queries).reshape(-1, heads * dim)
    batch = FakeBatch(contexts, q_lens)
    planned = attention_bf16.plan(batch, heads // kv_heads, kv_heads, torch.device(DEVICE))
    assert planned[4] == splits, planned
    out = attention_bf16.try_attention(packed.to(DEVICE), q_stride, batch, tables, k_pages, v_pages, heads, kv_heads, dim, scale, 0)
    torch.cuda.synchronize()
    from llmserver_b200.ops import gemm_bf16
    gemm_bf16.check_errors()
    want = torch.cat([plain_attention_rows(q.double(), k.double(), v.double(), scale, None, c - 1)
                      for q, k, v, c in zip(queries, dense_k, dense_v, contexts)])
    close(out, want, dtype, f"decode attention split {splits} ways")

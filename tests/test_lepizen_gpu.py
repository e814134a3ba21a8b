"""The Lepizen design in the engine against its plain implementation (tests/plain/lepizen_plain.py).

First every mechanism alone through its kernel (sink attention with values of their own size, the projection norm
with value blend and cache store, the GELU and scaled-add product epilogues, the soft cap), with inputs made so
that a lost sink, a far key or a blend left out shows; then whole models of six small configurations that differ
in every size and option, cut and batched in every way, both number formats.
"""
import copy
import json
import math
import os
import random

import numpy as np
import pytest
import torch

from helpers import batch_index, paged_cache, rel_error
from plain import lepizen_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
KERNEL_TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
MODEL_TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def _layer(heads, kv_heads, dim, vdim, scale, v_mix, ff):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": scale, "v_mix": v_mix},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _config(vocab, width, eps, mult, logit_scale, cap, layers):
    return {"architecture": "Lepizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "logit_scale": logit_scale, "logit_softcap": cap, "layers": layers}


CONFIGS = {
    # layers of unlike head counts and sizes; the first layer does not mix, one layer has no feed-forward
    "A": _config(200, 64, 1e-5, 0.5, 8.0, 20.0, [_layer(4, 2, 16, 32, 0.3, False, 96), _layer(4, 2, 32, 16, 0.2, True, None),
                                                  _layer(6, 2, 16, 16, 0.25, True, 80), _layer(4, 2, 32, 16, 0.15, True, 64)]),
    # what other models keep apart is equal or 1 here: as many kv heads as heads, values of the keys' size, no
    # residual multiplier, no logit scale, one mixing layer only (so nothing is ever blended)
    "B": _config(128, 96, 1e-6, 1.0, 1.0, 50.0, [_layer(3, 3, 32, 32, 0.18, True, 128), _layer(3, 3, 32, 32, 0.18, False, 128)]),
    # nothing a multiple of 8: the CUDA-core kernels serve both formats
    "C": _config(97, 100, 2e-5, 0.3, 2.5, 10.0, [_layer(5, 5, 20, 12, 0.22, True, 70), _layer(3, 1, 20, 12, 0.3, False, 30),
                                                  _layer(5, 5, 12, 12, 0.4, True, 70)]),
    # keys and values of 64: the TMA-fed and tcgen05 attention kernels, with their sinks
    "D": _config(300, 128, 1e-6, 0.4, 9.0, 12.0, [_layer(8, 2, 64, 64, 0.125, True, 192), _layer(8, 2, 64, 64, 0.125, True, 192)]),
    # keys of 128 and values of 64, four query heads on one kv head
    "E": _config(160, 128, 1e-6, 0.6, 5.0, 15.0, [_layer(4, 1, 128, 64, 0.09, True, 256), _layer(8, 1, 48, 64, 0.14, True, 64)]),
    # tensor-core head sizes beside an odd inner width and an odd vocabulary: the buffer that the attention and the
    # feed-forward share then has rows of an odd length
    "F": _config(131, 96, 1e-6, 0.7, 3.0, 25.0, [_layer(4, 2, 32, 16, 0.2, True, 77), _layer(2, 1, 16, 48, 0.3, False, 51)]),
}
SEEDS = {"A": 11, "B": 12, "C": 13, "D": 14, "E": 15, "F": 16}


@pytest.fixture(scope="module")
def ops():
    from aegean_tge_b200 import ops as module
    return module


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from aegean_tge_b200 import write_random_model
    out = {}
    for name, config in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"lepizen_{name}")
        write_random_model(str(folder), config, seed=SEEDS[name], dtype="float32")
        out[name] = str(folder)
    return out


def _read_weights(folder):
    """The safetensors file as numpy arrays (float32 and int32 tensors only), read here and not by the package."""
    with open(os.path.join(folder, "model.safetensors"), "rb") as handle:
        size = int.from_bytes(handle.read(8), "little")
        header = json.loads(handle.read(size))
        data = handle.read()
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        assert entry["dtype"] == "F32", (name, entry["dtype"])
        begin, end = entry["data_offsets"]
        out[name] = np.frombuffer(data[begin:end], dtype="<f4").reshape(entry["shape"]).copy()
    return out


def _to_bfloat16(array):
    return torch.from_numpy(array).to(torch.bfloat16).float().numpy()


@pytest.fixture(scope="module")
def oracle(folders):
    weights, cache = {}, {}

    def get(name, dtype, tokens, config=None):
        if (name, dtype) not in weights:
            w = _read_weights(folders[name])
            if dtype == "bfloat16":         # the engine holds matrices in bfloat16 and vectors in float32
                w = {k: (_to_bfloat16(v) if v.ndim == 2 else v) for k, v in w.items()}
            weights[(name, dtype)] = w
        key = (name, dtype, tuple(tokens), json.dumps(config, sort_keys=True) if config else "")
        if key not in cache:
            cache[key] = torch.from_numpy(plain.forward(config or CONFIGS[name], weights[(name, dtype)], list(tokens))).float()
        return cache[key]
    return get


def _tokens(name, count, salt=0):
    rnd = random.Random(SEEDS[name] * 1000 + salt)
    return [rnd.randrange(CONFIGS[name]["vocab"]) for _ in range(count)]


def _engine(folders, name, dtype, **kw):
    from aegean_tge_b200 import Engine
    kw.setdefault("context", 512)
    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_requests", 8)
    return Engine(folders[name], dtype=dtype, **kw)


def _portion(request, tokens, want=None):
    from aegean_tge_b200.engine import Portion
    return Portion(request, tokens, list(range(len(tokens))) if want is None else want)


# ---------------------------------------------------------------------------
# mechanisms, one by one
# ---------------------------------------------------------------------------
def _sink_attention_case(ops, dtype, heads, kv_heads, dim, vdim, q_lens, starts, sink_value=None, split=0, page_size=16,
                         force_simt=False, spike=None, decode_prefix=0):
    lengths = [s + n for s, n in zip(starts, q_lens)]
    k_pages, _, table, k_list, _ = paged_cache(lengths, kv_heads, dim, page_size, dtype, DEV, seed=5)
    _, v_pages, table_v, _, v_list = paged_cache(lengths, kv_heads, vdim, page_size, dtype, DEV, seed=5)
    assert torch.equal(table, table_v)
    positions, seq_of_token, q_start, start_pos = batch_index(q_lens, starts, DEV)
    T = sum(q_lens)
    gen = torch.Generator().manual_seed(23)
    buf = torch.randn(T, heads * dim + 40, generator=gen).to(dtype)
    sink = torch.randn(heads, generator=gen) * 2.0 if sink_value is None else torch.full((heads,), float(sink_value))
    scale = 1.3 / math.sqrt(dim)
    if spike is not None:
        seq, key_pos, head = spike          # one key of that request carries the last row's weight in this head
        row = sum(q_lens[:seq + 1]) - 1
        direction = k_list[seq][key_pos, head // (heads // kv_heads)].float()
        buf[row, head * dim:(head + 1) * dim] = (direction / direction.norm() * 80.0 / scale / direction.norm()).to(dtype)
    out = ops.attention(buf.to(DEV)[:, :heads * dim], k_pages, v_pages, table, q_start, start_pos, positions, seq_of_token,
                        len(q_lens), max(q_lens), max(lengths), heads, kv_heads, dim, scale, split_tokens=split,
                        force_simt=force_simt, decode_prefix=decode_prefix, sink=sink.to(DEV))
    ops.check_status()
    q = buf[:, :heads * dim].float().numpy().reshape(T, heads, dim)
    refs, begin = [], 0
    for s, (n, start) in enumerate(zip(q_lens, starts)):
        refs.append(plain.sink_attention(q[begin:begin + n], k_list[s].float().numpy(), v_list[s].float().numpy(),
                                         sink.numpy(), scale, start=start))
        begin += n
    ref = torch.from_numpy(np.concatenate(refs)).reshape(T, heads * vdim)
    assert tuple(out.shape) == (T, heads * vdim)
    return rel_error(out, ref), out, ref


SIZES = [(6, 2, 48, 16), (3, 1, 32, 64), (4, 4, 16, 16), (8, 2, 64, 64), (4, 1, 128, 128), (5, 5, 80, 32), (4, 2, 16, 256)]
CUTS = [([5, 1, 37, 2], [30, 150, 0, 63]), ([1, 1, 1], [0, 199, 64]), ([130], [0]), ([70, 3], [200, 15])]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", SIZES + [(2, 2, 100, 20), (3, 1, 24, 40)])
def test_sink_attention_on_the_cuda_cores(ops, dtype, heads, kv_heads, dim, vdim):
    for q_lens, starts in CUTS[:2]:
        err, _, _ = _sink_attention_case(ops, dtype, heads, kv_heads, dim, vdim, q_lens, starts, force_simt=True)
        assert err < KERNEL_TOL[dtype]


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", SIZES)
@pytest.mark.parametrize("q_lens,starts", CUTS)
@pytest.mark.parametrize("page_size", [16, 64])
def test_sink_attention_on_the_tensor_cores(ops, heads, kv_heads, dim, vdim, q_lens, starts, page_size):
    err, _, _ = _sink_attention_case(ops, torch.bfloat16, heads, kv_heads, dim, vdim, q_lens, starts, page_size=page_size)
    assert err < KERNEL_TOL[torch.bfloat16]


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(6, 2, 48, 16), (8, 2, 64, 64), (4, 1, 128, 128), (4, 2, 16, 256)])
@pytest.mark.parametrize("split", [64, 128, 192])
@pytest.mark.parametrize("q_lens,starts", [([1, 1, 1, 1], [700, 3, 255, 256]), ([40, 1], [300, 129]), ([300, 2], [1800, 0])])
def test_sink_attention_with_cut_keys_counts_the_sink_once(ops, heads, kv_heads, dim, vdim, split, q_lens, starts):
    """The keys cut into up to thirty splits that are merged: the sink must join the denominator once, not per split."""
    err, _, _ = _sink_attention_case(ops, torch.bfloat16, heads, kv_heads, dim, vdim, q_lens, starts, split=split,
                                     page_size=64, sink_value=3.0)
    assert err < KERNEL_TOL[torch.bfloat16]


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(6, 2, 48, 16), (8, 2, 64, 64), (4, 1, 128, 64)])
@pytest.mark.parametrize("page_size,split", [(16, 0), (64, 128), (64, 64)])
def test_single_tokens_at_the_head_of_a_mixed_step_keep_their_sinks(ops, heads, kv_heads, dim, vdim, page_size, split):
    """Nine single tokens deep in their contexts beside two prompt portions: the single tokens go to the decode
    kernel (their keys cut), the portions to the prompt kernel, both with the sink, one far key carrying a row."""
    q_lens = [1] * 9 + [37, 70]
    starts = [600, 0, 511, 512, 130, 64, 63, 1000, 257, 30, 200]
    err, _, _ = _sink_attention_case(ops, torch.bfloat16, heads, kv_heads, dim, vdim, q_lens, starts, split=split,
                                     page_size=page_size, sink_value=1.5, decode_prefix=9, spike=(0, 5, 0))
    assert err < KERNEL_TOL[torch.bfloat16]


@pytest.mark.parametrize("dtype,simt", [(torch.float32, True), (torch.bfloat16, True), (torch.bfloat16, False)])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(6, 2, 48, 16), (8, 2, 64, 64)])
def test_a_sink_left_out_would_show(ops, dtype, simt, heads, kv_heads, dim, vdim):
    """With a sink far above every score the output all but vanishes; with one far below it is plain attention."""
    _, high, _ = _sink_attention_case(ops, dtype, heads, kv_heads, dim, vdim, [9, 1], [40, 300], sink_value=40.0, force_simt=simt)
    err, low, ref = _sink_attention_case(ops, dtype, heads, kv_heads, dim, vdim, [9, 1], [40, 300], sink_value=-40.0, force_simt=simt)
    assert err < KERNEL_TOL[dtype]
    assert float(high.float().abs().max()) < 1e-6 * float(low.float().abs().max())
    err, mid, ref = _sink_attention_case(ops, dtype, heads, kv_heads, dim, vdim, [9, 1], [40, 300], sink_value=1.0, force_simt=simt)
    assert err < KERNEL_TOL[dtype]
    assert rel_error(mid, low.float().cpu()) > 0.01                           # the sink matters at this size


@pytest.mark.parametrize("dtype,simt", [(torch.float32, True), (torch.bfloat16, True), (torch.bfloat16, False)])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(6, 2, 48, 16), (8, 2, 64, 64), (4, 1, 128, 64)])
@pytest.mark.parametrize("q_lens,starts,key", [([1, 3], [900, 20], 7), ([1, 3], [900, 20], 63), ([1, 3], [900, 20], 64),
                                               ([200, 1], [700, 5], 3), ([1], [1023], 0), ([1], [1024], 1024)])
def test_sink_attention_reads_a_far_key(ops, dtype, simt, heads, kv_heads, dim, vdim, q_lens, starts, key):
    """One key far back (the first, one at a page's edge, the row's own) carries a head's weight against the sink
    and a thousand others: the output must be its value.  Single tokens and a prompt's last row."""
    err, out, ref = _sink_attention_case(ops, dtype, heads, kv_heads, dim, vdim, q_lens, starts, sink_value=2.0,
                                         force_simt=simt, spike=(0, key, heads - 1), page_size=64)
    assert err < KERNEL_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(6, 2, 48, 16), (3, 1, 32, 64), (5, 5, 20, 12), (8, 2, 64, 64), (300, 4, 8, 8)])
@pytest.mark.parametrize("blend", [None, 0.37])
def test_projection_norm_blend_and_store(ops, dtype, per_head, heads, kv_heads, dim, vdim, blend):
    """q and k normalised over the whole projection (or per head), v blended with another layer's, k and v stored."""
    q_lens, starts, page_size, eps = [5, 1, 37], [30, 150, 0], 16, 3e-4
    lengths = [s + n for s, n in zip(starts, q_lens)]
    k_pages, _, table, _, _ = paged_cache(lengths, kv_heads, dim, page_size, dtype, DEV, seed=3)
    _, v_pages, _, _, _ = paged_cache(lengths, kv_heads, vdim, page_size, dtype, DEV, seed=3)
    positions, seq_of_token, _, _ = batch_index(q_lens, starts, DEV)
    T = sum(q_lens)
    gen = torch.Generator().manual_seed(4)
    nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
    rows = (torch.randn(T, nq + nk + nv + 8, generator=gen) * 3.0).to(dtype)
    other = torch.randn(T, nv + 8, generator=gen).to(dtype)
    qw = torch.rand(dim if per_head else nq, generator=gen) + 0.5
    kw = torch.rand(dim if per_head else nk, generator=gen) + 0.5
    dev_rows = rows.to(DEV)
    lam = None if blend is None else torch.tensor([blend], dtype=torch.float32, device=DEV)
    ops.qk_norm_kv_store(dev_rows, qw.to(DEV), kw.to(DEV), eps, per_head, positions, seq_of_token, table, k_pages, v_pages,
                         heads, kv_heads, dim, vdim, v_other=None if blend is None else other.to(DEV)[:, :nv], blend=lam)
    ops.check_status()
    x = rows.float().numpy().astype(np.float64)
    if per_head:
        q_ref = plain.rms_norm(x[:, :nq].reshape(T, heads, dim), qw.numpy(), eps).reshape(T, nq)
        k_ref = plain.rms_norm(x[:, nq:nq + nk].reshape(T, kv_heads, dim), kw.numpy(), eps).reshape(T, nk)
    else:
        q_ref = plain.rms_norm(x[:, :nq], qw.numpy(), eps)
        k_ref = plain.rms_norm(x[:, nq:nq + nk], kw.numpy(), eps)
    v_ref = plain.blend_values(x[:, nq + nk:nq + nk + nv], None if blend is None else other.float().numpy()[:, :nv], blend or 0.0)
    tol = KERNEL_TOL[dtype]
    assert rel_error(dev_rows[:, :nq], torch.from_numpy(q_ref)) < tol
    assert rel_error(dev_rows[:, nq:nq + nk], torch.from_numpy(k_ref)) < tol
    assert rel_error(dev_rows[:, nq + nk:nq + nk + nv], torch.from_numpy(v_ref)) < tol
    assert torch.equal(dev_rows[:, nq + nk + nv:].cpu(), rows[:, nq + nk + nv:])           # nothing beyond the row's v
    begin = 0
    for s, (n, start) in enumerate(zip(q_lens, starts)):
        for i in range(n):
            pos = start + i
            page = int(table[s, pos // page_size])
            got_k = k_pages[page, :, pos % page_size, :].reshape(-1)
            got_v = v_pages[page, :, pos % page_size, :].reshape(-1)
            assert torch.equal(got_k, dev_rows[begin + i, nq:nq + nk])
            assert torch.equal(got_v, dev_rows[begin + i, nq + nk:nq + nk + nv])
        begin += n


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,width,up_rows", [(6, 2, 48, 16, 256, 0), (3, 1, 32, 64, 128, 200), (8, 2, 64, 64, 512, 2304),
                                                                 (28, 4, 128, 128, 512, 4104)])
@pytest.mark.parametrize("q_lens,starts", [([1, 1, 1], [30, 47, 0]), ([5, 1, 20], [30, 47, 0]), ([70, 58], [3, 16])])
@pytest.mark.parametrize("blend,deferred", [(None, False), (0.37, False), (0.6, True)])
def test_small_batch_product_with_norm_blend_store_and_gelu(ops, heads, kv_heads, dim, vdim, width, up_rows, q_lens, starts,
                                                             blend, deferred):
    """One product over the rows [q | k | v | up] whose partial sums one kernel adds, normalises, blends, stores and
    activates: against the same steps in float64, also from rows that still lack their norm factor."""
    page_size, eps = 16, 2e-4
    lengths = [s + n for s, n in zip(starts, q_lens)]
    k_pages, _, table, _, _ = paged_cache(lengths, kv_heads, dim, page_size, torch.bfloat16, DEV, seed=3)
    _, v_pages, _, _, _ = paged_cache(lengths, kv_heads, vdim, page_size, torch.bfloat16, DEV, seed=3)
    positions, seq_of_token, _, _ = batch_index(q_lens, starts, DEV)
    T = sum(q_lens)
    gen = torch.Generator().manual_seed(12)
    nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
    x = torch.randn(T, width, generator=gen).to(torch.bfloat16)
    w = (torch.randn(nq + nk + nv + up_rows, width, generator=gen) / math.sqrt(width)).to(torch.bfloat16)
    other = torch.randn(T, nv + 8, generator=gen).to(torch.bfloat16)
    qw, kw = torch.rand(nq, generator=gen) + 0.5, torch.rand(nk, generator=gen) + 0.5
    lam = None if blend is None else torch.tensor([blend], dtype=torch.float32, device=DEV)
    act = torch.zeros(T, up_rows + 8, dtype=torch.bfloat16, device=DEV) if up_rows else None
    given, factor = x.to(DEV), torch.ones(T, 1, dtype=torch.float64)
    if deferred:
        sums = torch.rand(3, T, generator=gen) * width
        given = ops.DeferredRows(x.to(DEV), sums.to(DEV), width, 1e-5)
        factor = (1.0 / torch.sqrt(sums.double().sum(0) / width + 1e-5))[:, None]
    qkv = ops.linear_qkv_norm_act_store(given, w.to(DEV), heads, kv_heads, dim, vdim, qw.to(DEV), kw.to(DEV), eps, positions,
                                        seq_of_token, table, k_pages, v_pages,
                                        v_other=None if blend is None else other.to(DEV)[:, :nv], blend=lam,
                                        act_out=None if act is None else act[:, :up_rows], activation=ops.GEMM_GELU)
    ops.check_status()
    assert qkv is not None and tuple(qkv.shape) == (T, nq + nk + nv)
    z = (x.double() @ w.double().T * factor).numpy()
    tol = KERNEL_TOL[torch.bfloat16]
    assert rel_error(qkv[:, :nq], torch.from_numpy(plain.rms_norm(z[:, :nq], qw.numpy(), eps))) < tol
    assert rel_error(qkv[:, nq:nq + nk], torch.from_numpy(plain.rms_norm(z[:, nq:nq + nk], kw.numpy(), eps))) < tol
    v_ref = plain.blend_values(z[:, nq + nk:nq + nk + nv], None if blend is None else other.float().numpy()[:, :nv], blend or 0.0)
    assert rel_error(qkv[:, nq + nk:], torch.from_numpy(v_ref)) < tol
    if up_rows:
        assert rel_error(act[:, :up_rows], torch.from_numpy(plain.gelu_erf(z[:, nq + nk + nv:]))) < tol
        assert float(act[:, up_rows:].abs().max()) == 0.0
    begin = 0
    for s, (n, start) in enumerate(zip(q_lens, starts)):
        for i in range(n):
            pos = start + i
            page = int(table[s, pos // page_size])
            assert torch.equal(k_pages[page, :, pos % page_size, :].reshape(-1), qkv[begin + i, nq:nq + nk])
            assert torch.equal(v_pages[page, :, pos % page_size, :].reshape(-1), qkv[begin + i, nq + nk:])
        begin += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(9, 260, 328), (150, 384, 704), (3, 97, 100), (700, 520, 264)])
@pytest.mark.parametrize("simt", [False, True])
def test_product_epilogues_gelu_and_scaled_add(ops, dtype, M, N, K, simt):
    gen = torch.Generator().manual_seed(6)
    x = torch.randn(M, K, generator=gen).to(dtype)
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K) * 2.0).to(dtype)
    z = x.double() @ w.double().T
    tol = KERNEL_TOL[dtype]
    erf = torch.from_numpy(plain.gelu_erf(z.numpy()))
    got = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_GELU, force_simt=simt)
    assert rel_error(got, erf) < tol
    tanh = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
    got = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_GELU_TANH, force_simt=simt)
    assert rel_error(got, tanh) < tol
    assert rel_error(erf, tanh) > 2 * KERNEL_TOL[torch.float32]     # the two forms are told apart in float32
    part = N // 3                                           # only the tail of the columns is activated
    got = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_GELU, force_simt=simt, act_from=part)
    assert rel_error(got, torch.cat([z[:, :part], erf[:, part:]], dim=1)) < tol
    stream = torch.randn(M, N, generator=gen)
    dev_stream = stream.to(DEV)
    ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_ADD_F32, out=dev_stream, force_simt=simt, alpha=0.3)
    assert rel_error(dev_stream, stream.double() + 0.3 * z) < tol
    got = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_STORE_F32, force_simt=simt, alpha=2.5)
    assert rel_error(got, 2.5 * z) < tol
    # a strided output, as when two parts write side by side into one buffer
    wide = torch.zeros(M, N + 16, dtype=dtype, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_GELU, out=wide[:, 16:], force_simt=simt)
    assert rel_error(wide[:, 16:], erf) < tol and float(wide[:, :16].abs().max()) == 0.0


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (8, 512, 512), (33, 520, 264), (128, 1024, 320), (140, 384, 192)])
@pytest.mark.parametrize("defer", [False, True])
def test_scaled_add_with_the_next_norm(ops, M, N, K, defer):
    """stream += alpha * product, then the next layer's norm, in the kernels that small batches use."""
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen) / math.sqrt(K)).to(torch.bfloat16)
    stream = torch.randn(M, N, generator=gen)
    gain = torch.rand(N, generator=gen) + 0.5
    dev_stream = stream.to(DEV)
    out = ops.linear_add_norm(x.to(DEV), w.to(DEV), None, dev_stream, gain.to(DEV), 1e-5, torch.bfloat16, defer=defer, alpha=0.3)
    if isinstance(out, ops.DeferredRows):
        out = out.complete()
    want = stream.double() + 0.3 * (x.double() @ w.double().T)
    assert rel_error(dev_stream, want) < 2e-3
    assert rel_error(out, torch.from_numpy(plain.rms_norm(want.numpy(), gain.numpy(), 1e-5))) < KERNEL_TOL[torch.bfloat16]


def test_soft_cap(ops):
    z = torch.linspace(-200.0, 200.0, 5 * 331).reshape(5, 331)
    got = ops.soft_cap(z.to(DEV).clone(), 25.0)
    assert rel_error(got, torch.from_numpy(plain.soft_cap(z.double().numpy(), 25.0))) < 1e-6
    assert float(got.abs().max()) <= 25.0


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_first_tokens(folders, oracle, ops, name, dtype):
    engine = _engine(folders, name, dtype)
    for length in (1, 2, 3, 7, 16, 64, 65, 130):
        tokens = _tokens(name, length, salt=length)
        logits = engine.runner.step([_portion("r", tokens)])
        engine.runner.finish("r")
        assert rel_error(logits, oracle(name, dtype, tokens)) < MODEL_TOL[dtype], (name, dtype, length)
    ops.check_status()
    engine.cache.check()


@pytest.mark.parametrize("name", ["A", "D"])
def test_each_mechanism_left_out_would_show(oracle, name):
    """The oracle without value mixing, with another residual multiplier, or without the cap differs from the
    model by far more than the tolerance: the model tests can tell."""
    tokens = _tokens(name, 40, salt=77)
    ref = oracle(name, "float32", tokens)
    for change in ("v_mix", "residual_mult", "logit_softcap", "scale"):
        other = copy.deepcopy(CONFIGS[name])
        if change == "v_mix":
            for layer in other["layers"]:
                layer["mixer"]["v_mix"] = False
        elif change == "scale":
            other["layers"][-1]["mixer"]["scale"] *= 1.5
        else:
            other[change] *= 1.5
        least = 100 * MODEL_TOL["float32"] if change == "scale" else MODEL_TOL["bfloat16"]
        assert rel_error(oracle(name, "float32", tokens, other), ref) > least, change


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token_decoding(folders, oracle, name, dtype):
    tokens = _tokens(name, 100, salt=1)
    ref = oracle(name, dtype, tokens)
    engine = _engine(folders, name, dtype)
    rows = [engine.runner.step([_portion("r", tokens[:68])])]
    for t in range(68, 100):
        rows.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
    got = torch.cat(rows)
    assert rel_error(got, ref) < MODEL_TOL[dtype]
    if dtype == "float32":
        whole = _engine(folders, name, dtype).runner.step([_portion("w", tokens)])
        assert float((got - whole).abs().max()) <= 1e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("page_size", [16, 64])
def test_portions_down_to_two_tokens(folders, oracle, name, dtype, page_size):
    tokens = _tokens(name, 150, salt=2)
    ref = oracle(name, dtype, tokens)
    engine = _engine(folders, name, dtype, page_size=page_size)
    cuts = [7, 2, 16, 3, 2, 30, 2, 17, 41, 1, 1, 26, 2]
    assert sum(cuts) == len(tokens)
    rows, pos = [], 0
    for count in cuts:
        rows.append(engine.runner.step([_portion("r", tokens[pos:pos + count])]))
        pos += count
    assert rel_error(torch.cat(rows), ref) < MODEL_TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("page_size,pool_tokens", [(16, 320), (64, 512)])
def test_unequal_requests_in_one_batch_on_pages_that_are_used_again(folders, oracle, ops, name, dtype, page_size, pool_tokens):
    """Up to four live requests, portions of some beside single tokens of others, a pool so small that pages of
    finished requests serve the next ones; every request's logits are those it gets alone."""
    lengths = {"a": 70, "b": 45, "c": 130, "d": 19, "e": 64, "f": 33, "g": 90}
    tokens = {r: _tokens(name, n, salt=ord(r)) for r, n in lengths.items()}
    engine = _engine(folders, name, dtype, max_tokens=pool_tokens, page_size=page_size)
    got, done = {r: [] for r in lengths}, {r: 0 for r in lengths}
    holders = {}                                  # page of the first group -> the requests that held it

    def run(step):
        logits = engine.runner.step([_portion(r, tokens[r][done[r]:done[r] + count]) for r, count in step])
        row = 0
        for r, count in step:
            got[r].append(logits[row:row + count])
            row += count
            done[r] += count
            for page in engine.cache.groups[0].tables[r]:
                holders.setdefault(page, set()).add(r)
            if done[r] == lengths[r]:
                engine.runner.finish(r)

    run([("a", 40), ("b", 3)])
    run([("a", 2), ("b", 40), ("c", 64), ("d", 1)])
    run([("a", 28), ("b", 2), ("c", 2), ("d", 16)])          # a and b end
    run([("c", 60), ("d", 2), ("e", 1), ("f", 30)])           # d ends; e and f take over pages
    for _ in range(3):
        run([("c", 1), ("e", 1), ("f", 1)])                   # f ends
    run([("c", 1), ("e", 58), ("g", 2)])
    run([("e", 2), ("g", 64)])                                # c ended before; e ends
    run([("g", 24)])
    ops.check_status()
    engine.cache.check()
    assert any(len(who) > 1 for who in holders.values()) and not engine.cache.live_requests()
    for r in lengths:
        assert done[r] == lengths[r]
        assert rel_error(torch.cat(got[r]), oracle(name, dtype, tokens[r])) < MODEL_TOL[dtype], (name, dtype, r)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D", "E"])
def test_long_decoding(folders, oracle, name, dtype):
    """Three tokens of prompt, then 300 single tokens through the decode graphs, over several pages."""
    tokens = _tokens(name, 303, salt=5)
    ref = oracle(name, dtype, tokens)
    engine = _engine(folders, name, dtype)
    rows = [engine.runner.step([_portion("r", tokens[:3])])]
    for t in range(3, len(tokens)):
        rows.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
    assert rel_error(torch.cat(rows), ref) < MODEL_TOL[dtype]
    assert engine.runner.graph_replays > 0


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_scheduler(folders, oracle, name):
    """``Engine.generate`` (scheduler, portions of 16, sampler) gives the plain model's greedy continuation."""
    engine = _engine(folders, name, "float32", chunk=16, max_batch_tokens=48)
    prompts = [_tokens(name, n, salt=40 + n) for n in (5, 37, 1, 70)]
    outputs = engine.generate(prompts, n=12)
    for prompt, produced in zip(prompts, outputs):
        sequence = list(prompt)
        for token in produced:
            logits = oracle(name, "float32", sequence)[-1]
            best = int(torch.argmax(logits))
            if token != best:          # only a tie within rounding may differ
                assert float(logits[best] - logits[token]) < 1e-4 * float(logits.abs().max()), (name, len(sequence))
            sequence.append(int(token))
        assert len(produced) == 12
    assert not engine.cache.live_requests()
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_of_a_lepizen_model(folders, oracle, tmp_path, dtype):
    """bin/trace_run as a subprocess: two requests, portions and single tokens in one batch, a slot given back."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a, b = _tokens("A", 30, salt=90), _tokens("A", 9, salt=91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[20:21], "want": [0]}, {"id": "b", "tokens": b[:7], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [1]}, {"id": "a", "tokens": a[21:], "want": [8]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    run = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["A"], "--dtype", dtype,
                          "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref_a, ref_b = oracle("A", dtype, a), oracle("A", dtype, b)
    want = {0: ref_a[[0, 19]], 1: ref_a[[20]], 2: torch.cat([ref_b[[8]], ref_a[[29]]])}
    for step, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(ref.shape))
        assert rel_error(got, ref) < MODEL_TOL[dtype]


def test_command_line_serves_the_design(folders, capsys):
    """`tge generate`, `tge bench decode / prefill / mixed` and `tge plan` with a Lepizen folder: the commands know no design."""
    from aegean_tge_b200.cli import main
    assert main(["generate", "--model", folders["D"], "--tokens", "5 17 3", "--n", "6", "--print-ids", "--context", "128"]) == 0
    out = capsys.readouterr().out
    assert "prefill  :" in out and "decode   :" in out and len(out.split("ids      :")[1].split()) == 6
    common = ["--model", folders["D"], "--context", "512", "--max-requests", "12"]
    assert main(["bench", "decode", *common, "--batch", "3", "--prompt-len", "40", "--n", "4"]) == 0
    assert main(["bench", "prefill", *common, "--prompt-len", "100", "--repeat", "1"]) == 0
    assert main(["bench", "mixed", *common, "--batch", "9", "--prompt-len", "40", "--portion", "70", "--timeline"]) == 0
    out = capsys.readouterr().out
    assert "decode   : batch 3 at context 40" in out and "attention_decode" in out
    assert main(["plan", "--model", folders["A"], "--context", "256", "--sessions", "2"]) == 0
    assert "kv       :" in capsys.readouterr().out


@pytest.mark.parametrize("dtype", DTYPES)
def test_sampled_generation_with_requests_that_come_and_go(folders, dtype):
    """Twelve requests with temperature, top-k and top-p samplers through six slots and a small pool: all finish,
    the same seeds give the same tokens whatever shared a step with what, every page comes back."""
    from aegean_tge_b200 import SamplingParams
    prompts = [_tokens("A", 3 + 11 * i, salt=300 + i) for i in range(12)]
    params = [SamplingParams(temperature=0.8, top_k=(0, 20, 50)[i % 3], top_p=(1.0, 0.9)[i % 2], seed=40 + i) for i in range(12)]
    outputs = []
    for slots, budget, chunk in ((6, 64, 16), (3, 256, 64)):
        engine = _engine(folders, "A", dtype, max_requests=slots, max_batch_tokens=budget, chunk=chunk, max_tokens=640)
        outputs.append(engine.generate(prompts, n=10, sampling=params))
        assert all(len(row) == 10 for row in outputs[-1]) and not engine.cache.live_requests()
        engine.cache.check()
    if dtype == "float32":
        assert outputs[0] == outputs[1]

"""Convenience wrappers that call the C ABI on torch CUDA tensors (torch is only the device allocator and stream
provider here): one function per entry point, allocating the outputs.  Used by the tests, the smoke check and the
single-kernel benchmark cases; the graph path (compiler / executor) does not go through this module."""
import numpy as np
import torch

from . import capi

DT = {torch.float32: capi.F32, torch.float16: capi.FP16, torch.bfloat16: capi.BF16,
      torch.int32: capi.I32, torch.int64: capi.I64, torch.int8: capi.I8, torch.uint8: capi.U8, torch.int16: capi.I16, torch.bool: capi.BOOL}


def ptr(t):
    return 0 if t is None else t.data_ptr()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def stream():
    return torch.cuda.current_stream().cuda_stream


def rms_norm(x, w, eps, residual=None):
    y = torch.empty_like(x)
    p = capi.RmsNormParams(DT[x.dtype], x.numel() // x.shape[-1], x.shape[-1], eps, int(residual is not None))
    if residual is None:
        capi.call("rms_norm", p, [ptr(x), ptr(w)], [ptr(y)], stream=stream())
        return y
    s = torch.empty_like(x)
    capi.call("rms_norm", p, [ptr(x), ptr(w), ptr(residual)], [ptr(y), ptr(s)], stream=stream())
    return y, s


def softmax(x, axis):
    axis %= x.dim()
    pre = int(np.prod(x.shape[:axis], dtype=np.int64))
    post = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    y = torch.empty_like(x)
    capi.call("softmax", capi.SoftmaxParams(DT[x.dtype], pre, x.shape[axis], post), [ptr(x)], [ptr(y)], stream=stream())
    return y


def topk(x, k, softmax=False):
    rows, n = x.shape
    vals = torch.empty(rows, k, dtype=torch.float32 if softmax else x.dtype, device=x.device)
    idx = torch.empty(rows, k, dtype=torch.int64, device=x.device)
    capi.call("topk", capi.TopkParams(DT[x.dtype], rows, n, k, int(softmax)), [ptr(x)], [ptr(vals), ptr(idx)], stream=stream())
    return vals, idx


def topk_sample(x, k, temperature, seed, step):
    rows, n = x.shape
    st = torch.tensor([step], dtype=torch.int64, device=x.device)
    tok = torch.empty(rows, dtype=torch.int64, device=x.device)
    capi.call("topk_sample", capi.TopkSampleParams(DT[x.dtype], rows, n, k, temperature, seed), [ptr(x), ptr(st)], [ptr(tok)], stream=stream())
    return tok


def gather(data, idx, axis):
    prefix = int(np.prod(data.shape[:axis], dtype=np.int64))
    postfix = int(np.prod(data.shape[axis + 1:], dtype=np.int64)) * data.element_size()
    out = torch.empty(tuple(data.shape[:axis]) + tuple(idx.shape) + tuple(data.shape[axis + 1:]), dtype=data.dtype, device=data.device)
    p = capi.GatherParams(prefix, data.shape[axis], idx.numel(), postfix, DT[idx.dtype])
    capi.call("gather", p, [ptr(data), ptr(idx)], [ptr(out)], stream=stream())
    return out


def _bstrides(shape, out_shape):
    pad = (1,) * (len(out_shape) - len(shape)) + tuple(shape)
    st, acc = [0] * len(out_shape), 1
    for d in range(len(out_shape) - 1, -1, -1):
        st[d] = 0 if pad[d] == 1 and out_shape[d] != 1 else acc
        acc *= pad[d]
    return st


def _pad4(v, fill):
    return [fill] * (4 - len(v)) + list(v)


def binary(op, a, b, check=True):
    shape = torch.broadcast_shapes(a.shape, b.shape)
    y = torch.empty(shape, dtype=a.dtype, device=a.device)
    p = capi.BinaryParams()
    p.op, p.dtype = op, DT[a.dtype]
    p.shape[:] = _pad4(shape, 1)
    p.a_stride[:] = _pad4(_bstrides(a.shape, shape), 0)
    p.b_stride[:] = _pad4(_bstrides(b.shape, shape), 0)
    rc = capi.call("binary", p, [ptr(a), ptr(b)], [ptr(y)], stream=stream(), check=check)
    return y if check else (rc, y)


def unary(op, x):
    y = torch.empty_like(x)
    capi.call("unary", capi.UnaryParams(op, DT[x.dtype], x.numel()), [ptr(x)], [ptr(y)], stream=stream())
    return y


def where(c, a, b):
    shape = torch.broadcast_shapes(c.shape, a.shape, b.shape)
    y = torch.empty(shape, dtype=a.dtype, device=a.device)
    p = capi.WhereParams()
    p.dtype = DT[a.dtype]
    p.shape[:] = _pad4(shape, 1)
    p.c_stride[:] = _pad4(_bstrides(c.shape, shape), 0)
    p.a_stride[:] = _pad4(_bstrides(a.shape, shape), 0)
    p.b_stride[:] = _pad4(_bstrides(b.shape, shape), 0)
    capi.call("where", p, [ptr(c), ptr(a), ptr(b)], [ptr(y)], stream=stream())
    return y


def transpose(x, perm):
    y = torch.empty([x.shape[i] for i in perm], dtype=x.dtype, device=x.device)
    p = capi.TransposeParams()
    p.elem_bytes, p.rank = x.element_size(), x.dim()
    p.in_shape[:] = list(x.shape) + [1] * (4 - x.dim())
    p.perm[:] = list(perm) + [0] * (4 - x.dim())
    capi.call("transpose", p, [ptr(x)], [ptr(y)], stream=stream())
    return y


def _as_3d(shape, axis):
    axis %= len(shape)
    return int(np.prod(shape[:axis], dtype=np.int64)), int(shape[axis]), int(np.prod(shape[axis + 1:], dtype=np.int64))


def concat(xs, axis):
    axis %= xs[0].dim()
    outer, _, inner = _as_3d(xs[0].shape, axis)
    shape = list(xs[0].shape)
    shape[axis] = sum(int(x.shape[axis]) for x in xs)
    y = torch.empty(shape, dtype=xs[0].dtype, device=xs[0].device)
    p = capi.ConcatParams()
    p.elem_bytes, p.n_parts, p.outer, p.inner = xs[0].element_size(), len(xs), outer, inner
    for i, x in enumerate(xs):
        p.axis_len[i] = int(x.shape[axis])
    capi.call("concat", p, [ptr(x) if x.numel() else 0 for x in xs], [ptr(y)], stream=stream())
    return y


def split(x, sizes, axis):
    axis %= x.dim()
    outer, _, inner = _as_3d(x.shape, axis)
    ys = []
    for n in sizes:
        shape = list(x.shape)
        shape[axis] = n
        ys.append(torch.empty(shape, dtype=x.dtype, device=x.device))
    p = capi.ConcatParams()
    p.elem_bytes, p.n_parts, p.outer, p.inner = x.element_size(), len(sizes), outer, inner
    for i, n in enumerate(sizes):
        p.axis_len[i] = n
    capi.call("split", p, [ptr(x)], [ptr(y) if y.numel() else 0 for y in ys], stream=stream())
    return ys


def slice_(x, starts, steps, lengths, check=True):
    y = torch.empty(list(lengths), dtype=x.dtype, device=x.device)
    p = capi.SliceParams()
    p.elem_bytes, p.rank = x.element_size(), x.dim()
    for d in range(x.dim()):
        p.in_shape[d], p.start[d], p.step[d], p.length[d] = int(x.shape[d]), int(starts[d]), int(steps[d]), int(lengths[d])
    rc = capi.call("slice", p, [ptr(x)], [ptr(y)], stream=stream(), check=check)
    return y if check else (rc, y)


def expand(x, shape):
    y = torch.empty(list(shape), dtype=x.dtype, device=x.device)
    p = capi.ExpandParams()
    p.elem_bytes, p.rank = x.element_size(), len(shape)
    ins = [1] * (len(shape) - x.dim()) + list(x.shape)
    for d in range(len(shape)):
        p.in_shape[d], p.out_shape[d] = int(ins[d]), int(shape[d])
    capi.call("expand", p, [ptr(x)], [ptr(y)], stream=stream())
    return y


CAST_CODE = {torch.float32: capi.F32, torch.float64: capi.F64, torch.float16: capi.FP16, torch.bfloat16: capi.BF16, torch.int8: capi.I8,
             torch.uint8: capi.U8, torch.int16: capi.I16, torch.int32: capi.I32, torch.int64: capi.I64, torch.bool: capi.BOOL}


def cast(x, to):
    y = torch.empty(x.shape, dtype=to, device=x.device)
    p = capi.CastParams(CAST_CODE[x.dtype], CAST_CODE[to], x.numel())
    capi.call("cast", p, [ptr(x)], [ptr(y)], stream=stream())
    return y


def rope(x, pos, theta=10000.0):
    y = torch.empty_like(x)
    t, h, d = x.shape
    capi.call("rope", capi.RopeParams(DT[x.dtype], t, h, d, theta), [ptr(x), ptr(pos)], [ptr(y)], stream=stream())
    return y


def mat_mul(a, b, c=None, trans_a=False, trans_b=False, alpha=1.0, beta=1.0, force=0):
    """2-D or batched with equal / broadcast (size-1 or missing) leading dims flattened to one batch axis."""
    m = a.shape[-1] if trans_a else a.shape[-2]
    k = a.shape[-2] if trans_a else a.shape[-1]
    n = b.shape[-2] if trans_b else b.shape[-1]
    ba = int(np.prod(a.shape[:-2], dtype=np.int64))
    bb = int(np.prod(b.shape[:-2], dtype=np.int64))
    batch = max(ba, bb)
    assert ba in (1, batch) and bb in (1, batch)
    lead = a.shape[:-2] if ba >= bb else b.shape[:-2]
    y = torch.empty(tuple(lead) + (m, n), dtype=a.dtype, device=a.device)
    p = capi.MatMulParams()
    p.dtype, p.m, p.n, p.k = DT[a.dtype], m, n, k
    p.trans_a, p.trans_b, p.alpha, p.beta = int(trans_a), int(trans_b), alpha, beta
    p.batch = batch
    p.stride_a = m * k if ba == batch and batch > 1 else 0
    p.stride_b = k * n if bb == batch and batch > 1 else 0
    p.stride_y = m * n
    p.force_kernel = force
    if c is not None:
        p.has_bias = 1
        cs = _bstrides(c.shape, (m, n))
        p.bias_row_stride, p.bias_col_stride = cs[0], cs[1]
        p.stride_c = 0
    nws = capi.workspace("mat_mul", p)
    ws = torch.zeros(max(nws, 1), dtype=torch.uint8, device=a.device)
    capi.call("mat_mul", p, [ptr(a), ptr(b), ptr(c)], [ptr(y)], ws=ptr(ws) if nws else 0, stream=stream())
    torch.cuda.current_stream().synchronize()  # the workspace is released on return
    return y


def kv_layout(n_kv, d, max_seq=0, page=0, max_blocks=0, n_blocks=0):
    return capi.KvLayout(n_kv, d, max_seq, page, max_blocks, n_blocks)


def linear(x, w, g=None, eps=1e-6, residual=None, epilogue=0, n_heads=0, kv=None, positions=None, table=None,
           k_cache=None, v_cache=None, theta=10000.0, check=True, tokens_per_seq=0):
    m, k = x.shape
    n = w.shape[0]
    p = capi.LinearParams()
    p.tokens_per_seq = tokens_per_seq
    p.dtype, p.m, p.n, p.k = DT[x.dtype], m, n, k
    p.prologue, p.epilogue, p.epsilon, p.n_heads, p.theta = int(g is not None), epilogue, eps, n_heads, theta
    if kv is not None:
        p.kv = kv
    if epilogue == 2:
        y = torch.empty(m, n // 2, dtype=x.dtype, device=x.device)
    elif epilogue == 3:
        y = torch.empty(m, n_heads * kv.head_dim, dtype=x.dtype, device=x.device)
    else:
        y = torch.empty(m, n, dtype=x.dtype, device=x.device)
    nws = capi.workspace("linear", p)
    ws = torch.zeros(max(nws, 1), dtype=torch.uint8, device=x.device)
    rc = capi.call("linear", p, [ptr(x), ptr(w), ptr(g), ptr(residual), ptr(positions), ptr(table)],
                   [ptr(y), ptr(k_cache), ptr(v_cache)], ws=ptr(ws) if nws else 0, stream=stream(), check=check)
    if nws:
        torch.cuda.current_stream().synchronize()  # the workspace is released on return
    return y if check else (rc, y)


def attention(q, k, v, past=None, k_cache=None, v_cache=None):
    N, nH, S, D = q.shape
    o = torch.empty_like(q)
    has_cache = k_cache is not None
    p = capi.AttentionParams(DT[q.dtype], N, nH, k.shape[1], S, D, k_cache.shape[2] if has_cache else S, int(has_cache))
    pt = None if past is None else torch.tensor([past], dtype=torch.int64, device=q.device)
    capi.call("attention", p, [ptr(q), ptr(k), ptr(v), ptr(pt), ptr(k_cache), ptr(v_cache)],
              [ptr(o), ptr(k_cache), ptr(v_cache)], stream=stream())
    return o


def attn_decode(q, k_cache, v_cache, lens, kv, max_len, table=None, ws=None):
    B, nH, D = q.shape
    p = capi.AttnDecodeParams(DT[q.dtype], B, nH, max_len, kv)
    if ws is None:
        ws = torch.zeros(capi.workspace("attn_decode", p), dtype=torch.uint8, device=q.device)
    o = torch.empty_like(q)
    capi.call("attn_decode", p, [ptr(q), ptr(k_cache), ptr(v_cache), ptr(lens), ptr(table)], [ptr(o)], ws=ptr(ws), stream=stream())
    return o, ws

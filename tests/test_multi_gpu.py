"""Two ranks on two GPUs of one box: the peer-memory all-reduce against the reference's own vector and numpy, and a
tensor-parallel decode step against the unsharded oracle.  One process per GPU; IPC handles travel over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _exchange(handle: bytes):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, handle)
    return out


def _worker(rank, world, port, q, algo):
    try:
        # RG_B200_AR_ALGO picks the all-reduce variant (1 = one-shot push, 2 = two-shot); the library reads it once
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", RG_B200_AR_ALGO=algo)
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from refactorgraph_b200 import capi
        from refactorgraph_b200.llama import LlamaConfig, decode_step_graph_batched, seeded_weights, shard_config, shard_weights, weight_inputs
        from _decode_oracle import KvHistory, oracle_decode_step_rounded
        comm = capi.Comm(world, rank, 1 << 20, exchange=_exchange)
        res = {}
        # (1) the reference's all-reduce vector (src/04kernel/test/kernels/all_reduce/test_allreduce_nccl.cpp:44-47)
        x = torch.tensor([2.0, 3.0] if rank == 0 else [5.0, 6.0], device="cuda")
        y = torch.empty_like(x)
        comm.all_reduce(capi.F32, 0, 2, x.data_ptr(), y.data_ptr())
        torch.cuda.synchronize()
        res["kat"] = y.cpu().tolist() == [7.0, 9.0]
        # (2) every op / dtype on seeded data, ragged length, many calls in a row (slot reuse)
        ok = True
        for it, (op, dt, n) in enumerate([(0, torch.float32, 100003), (1, torch.float16, 65536), (2, torch.bfloat16, 777),
                                          (3, torch.float32, 8), (4, torch.float32, 4096), (0, torch.float16, 131072)] * 3):
            gens = [torch.Generator().manual_seed(100 * it + r) for r in range(world)]
            parts = [torch.randn(n, generator=g).to(dt) for g in gens]
            xs = parts[rank].cuda()
            ys = torch.empty_like(xs)
            code = {torch.float32: capi.F32, torch.float16: capi.FP16, torch.bfloat16: capi.BF16}[dt]
            comm.all_reduce(code, op, n, xs.data_ptr(), ys.data_ptr())
            torch.cuda.synchronize()
            f = [p.float() for p in parts]
            want = {0: f[0] + f[1], 1: (f[0] + f[1]) / 2, 2: torch.minimum(f[0], f[1]), 3: torch.maximum(f[0], f[1]), 4: f[0] * f[1]}[op].to(dt)
            ok = ok and torch.equal(ys.cpu(), want)
        res["ops"] = ok
        # (2b) the integer and double types the reference's NCCL kernel accepts: combined in their own type, bit-exact
        ok = True
        for it, (op, ndt, code, n) in enumerate([(0, np.int32, capi.I32, 5000), (0, np.uint8, capi.U8, 4099), (2, np.int8, capi.I8, 333),
                                                 (3, np.int64, capi.I64, 1025), (4, np.uint32, capi.U32, 64), (1, np.int32, capi.I32, 77),
                                                 (0, np.float64, capi.F64, 2049), (1, np.float64, capi.F64, 16), (4, np.int64, capi.I64, 9)]):
            rngs = [np.random.default_rng(1000 + 10 * it + r) for r in range(world)]
            if np.issubdtype(ndt, np.floating):
                parts = [g.standard_normal(n).astype(ndt) for g in rngs]
            else:
                info = np.iinfo(ndt)
                parts = [g.integers(info.min, info.max, n, dtype=ndt, endpoint=True) for g in rngs]
            xs = torch.from_numpy(parts[rank].view(np.uint8)).cuda()
            ys = torch.zeros_like(xs)
            comm.all_reduce(code, op, n, xs.data_ptr(), ys.data_ptr())
            torch.cuda.synchronize()
            a, b = parts
            with np.errstate(over="ignore"):
                if np.issubdtype(ndt, np.floating):
                    want = {0: a + b, 1: (a + b) * 0.5, 2: np.minimum(a, b), 3: np.maximum(a, b), 4: a * b}[op]
                else:    # sums and products wrap in the element type; Avg divides the wrapped sum (C++ division truncates toward zero)
                    ssum = (a + b).astype(ndt)
                    want = {0: ssum, 1: np.trunc(ssum / 2).astype(ndt) if np.issubdtype(ndt, np.signedinteger) else ssum // 2,
                            2: np.minimum(a, b), 3: np.maximum(a, b), 4: (a * b).astype(ndt)}[op]
            ok = ok and np.array_equal(ys.cpu().numpy().view(ndt)[:n], want.astype(ndt))
        res["int_ops"] = ok
        # (2c) all-reduce + residual + RMSNorm in one launch: the same bits as the all-reduce followed by the norm kernel
        import _ops as ops
        ok = True
        for it, (dt, rows, dim, with_res) in enumerate([(torch.float16, 16, 8192, True), (torch.bfloat16, 5, 512, True), (torch.float16, 3, 4096, False),
                                                        (torch.bfloat16, 16, 1024, True), (torch.float16, 2, 16384, True), (torch.float16, 7, 136, False)] * 2):
            gens = [torch.Generator().manual_seed(5000 + 10 * it + r) for r in range(world)]
            parts = [torch.randn(rows, dim, generator=g).to(dt) for g in gens]
            gw = torch.Generator().manual_seed(77 + it)
            res_t = torch.randn(rows, dim, generator=gw).to(dt).cuda() if with_res else None
            wn = (1.0 + 0.1 * torch.randn(dim, generator=gw)).to(dt).cuda()
            xs = parts[rank].cuda()
            code = capi.FP16 if dt == torch.float16 else capi.BF16
            y0 = torch.empty_like(xs)
            comm.all_reduce(code, 0, rows * dim, xs.data_ptr(), y0.data_ptr(), residual=res_t.data_ptr() if with_res else 0)
            n0 = ops.rms_norm(y0, wn, 1e-5)
            y1, n1 = torch.zeros_like(xs), torch.zeros_like(xs)
            comm.all_reduce_norm(code, rows, dim, 1e-5, xs.data_ptr(), wn.data_ptr(), y1.data_ptr(), n1.data_ptr(), residual=res_t.data_ptr() if with_res else 0)
            torch.cuda.synchronize()
            ok = ok and torch.equal(y0.view(torch.int16), y1.view(torch.int16)) and torch.equal(n0.view(torch.int16), n1.view(torch.int16))
        res["ar_norm"] = ok
        # (2d) row-parallel product whose epilogue is the sending half of the all-reduce + the receiving half: the same bits as
        # the tcgen05 product followed by the all-reduce (unsplit, k-split and stream-K plans; with and without residual)
        ok = True
        for it, (dt, m, n, k, with_res) in enumerate([(torch.float16, 16, 8192, 1024, True), (torch.float16, 16, 8192, 3584, True), (torch.bfloat16, 32, 4096, 4096, False),
                                                      (torch.float16, 64, 1024, 512, True), (torch.bfloat16, 5, 136, 64, False), (torch.float16, 16, 4096, 11008, True)] * 2):
            gx = torch.Generator().manual_seed(9000 + 10 * it + rank)
            xs = torch.randn(m, k, generator=gx).to(dt).cuda()
            wt = (0.05 * torch.randn(n, k, generator=gx)).to(dt).cuda()
            gr = torch.Generator().manual_seed(9500 + it)
            res_t = torch.randn(m, n, generator=gr).to(dt).cuda() if with_res else None
            code = capi.FP16 if dt == torch.float16 else capi.BF16
            p = capi.MatMulParams()
            p.dtype, p.m, p.n, p.k, p.trans_b, p.alpha, p.beta, p.batch, p.stride_y, p.force_kernel = code, m, n, k, 1, 1.0, 0.0, 1, m * n, 3
            nws = capi.workspace("mat_mul", p)
            wsb = torch.zeros(max(nws, 1), dtype=torch.uint8, device="cuda")
            y_part = torch.empty(m, n, dtype=dt, device="cuda")
            rc = capi.call("mat_mul", p, [xs.data_ptr(), wt.data_ptr(), 0], [y_part.data_ptr()], ws=wsb.data_ptr() if nws else 0, check=False)
            if rc != capi.OK:       # a shape the tcgen05 kernel does not take has no fused form either
                continue
            y0 = torch.empty_like(y_part)
            comm.all_reduce(code, 0, m * n, y_part.data_ptr(), y0.data_ptr(), residual=res_t.data_ptr() if with_res else 0)
            y1 = torch.zeros_like(y_part)
            p.force_kernel = 0
            comm.mat_mul_push(p, xs.data_ptr(), wt.data_ptr(), ws=wsb.data_ptr() if nws else 0)
            comm.all_reduce_recv(code, m * n, y1.data_ptr(), residual=res_t.data_ptr() if with_res else 0)
            torch.cuda.synchronize()
            ok = ok and torch.equal(y0.view(torch.int16), y1.view(torch.int16))
        res["mm_push"] = ok
        # (3) tensor-parallel decode step vs the unsharded oracle
        cfg = LlamaConfig(layers=2, hidden=512, heads=8, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=128, batch=16)
        rng = np.random.default_rng(3)
        w16 = seeded_weights(cfg, 0, np.float16)
        w16["lm_head"] = (0.2 * rng.standard_normal(w16["lm_head"].shape)).astype(np.float16)
        B = cfg.batch
        past = rng.integers(1, 100, (B,)).astype(np.int64)
        kc = [rng.standard_normal((B, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
        vc = [rng.standard_normal((B, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
        token = rng.integers(0, cfg.vocab, (B,)).astype(np.int64)
        # the oracle's tensor-parallel restatement: per-rank partial products rounded to fp16, summed in fp32 in rank order
        r16 = lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
        kh = [[KvHistory(kc[l][b], past[b]) for b in range(B)] for l in range(cfg.layers)]
        vh = [[KvHistory(vc[l][b], past[b]) for b in range(B)] for l in range(cfg.layers)]
        want_logits = [oracle_decode_step_rounded(cfg, {k: v.astype(np.float32) for k, v in w16.items()}, kh, vh, token, past, r16, world=world)]
        sc, kr = shard_config(cfg, world), cfg.kv_heads // world
        ws = shard_weights(cfg, w16, world, rank)
        g, index = decode_step_graph_batched(sc, world=world)
        ex = g.compiler().compile("cuda", "flat", [])
        ex.set_communicator(comm.address)
        for name, _ in weight_inputs(sc):
            ex.set_input(index[name], np.ascontiguousarray(ws[name]))
        for l in range(cfg.layers):
            ex.set_input(index[f"l{l}.k_cache"], np.ascontiguousarray(kc[l][:, rank * kr:(rank + 1) * kr]))
            ex.set_input(index[f"l{l}.v_cache"], np.ascontiguousarray(vc[l][:, rank * kr:(rank + 1) * kr]))
        ex.set_input(index["token"], token)
        ex.set_input(index["pos"], past)
        ex.set_input(index["lens"], past + 1)
        good = True
        for s in range(2):
            dist.barrier()
            ex.run()          # second run = CUDA-graph replay with the sequence number advancing on the device
            logits = ex.get_output(index["logits"]).astype(np.float32)
            if s == 0:
                good = good and np.allclose(logits, want_logits[0], atol=2e-2, rtol=1e-2)
            gathered = [None] * world
            dist.all_gather_object(gathered, logits.tobytes())
            good = good and gathered[0] == gathered[1]      # bit-identical logits on both ranks
        res["tp"] = bool(good)
        # (3b) the same graph through the fusion pass with an opt-in fused node (all-reduce + RMSNorm, or product + all-reduce,
        # by the all-reduce variant under test, so both get a run); same tolerance, ranks agree
        knob, node = ("RG_B200_FUSE_AR_NORM", "AllReduceNorm") if algo == "1" else ("RG_B200_FUSE_MM_AR", "MatMulAllReduce")
        os.environ[knob] = "1"
        assert g.compiler().plan(["fuse"]).count(node) == 2 * cfg.layers
        exf = g.compiler().compile("cuda", "flat", ["fuse"])
        exf.set_communicator(comm.address)
        for name, _ in weight_inputs(sc):
            exf.set_input(index[name], np.ascontiguousarray(ws[name]))
        for l in range(cfg.layers):
            exf.set_input(index[f"l{l}.k_cache"], np.ascontiguousarray(kc[l][:, rank * kr:(rank + 1) * kr]))
            exf.set_input(index[f"l{l}.v_cache"], np.ascontiguousarray(vc[l][:, rank * kr:(rank + 1) * kr]))
        exf.set_input(index["token"], token)
        exf.set_input(index["pos"], past)
        exf.set_input(index["lens"], past + 1)
        dist.barrier()
        exf.run()
        lf = exf.get_output(index["logits"]).astype(np.float32)
        gathered = [None] * world
        dist.all_gather_object(gathered, lf.tobytes())
        res["tp_fused"] = bool(np.allclose(lf, want_logits[0], atol=2e-2, rtol=1e-2) and gathered[0] == gathered[1])
        dist.barrier()
        del exf
        res["status"] = comm.status() == capi.OK
        dist.barrier()
        del ex
        comm.destroy()
        dist.destroy_process_group()
        q.put((rank, res))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs on one box")
@pytest.mark.parametrize("algo", ["1", "2"])
def test_two_ranks_all_reduce_and_tensor_parallel_decode(algo):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, algo)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    for r in range(2):
        assert "error" not in results[r], results[r].get("error")
        assert results[r] == {"kat": True, "ops": True, "int_ops": True, "ar_norm": True, "mm_push": True, "tp": True, "tp_fused": True, "status": True}, results[r]

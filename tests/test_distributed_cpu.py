"""Multi-process logic on CPU ranks (gloo, world size 2, 127.0.0.1): collectives, TP/SP, PP 1F1B, ring attention,
expert parallel MoE, FSDP wrappers, DTensor, and failure detection when a rank leaves."""
import json
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PRELUDE = r'''
import json, os, sys, math, torch
sys.path.insert(0, %(root)r)
import torch.distributed as dist
import litetorch_b200 as lt
from litetorch_b200.core import _unwrap
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
pg = lt.distributed.init_process_group(rank, world, "127.0.0.1", int(os.environ["MASTER_PORT"]), backend="gloo")
def done(**kw):
    if rank == 0:
        print("RESULT " + json.dumps(kw))
    dist.barrier()
    pg.shutdown()
'''


def run_ranks(body: str, nproc: int = 2, port: int = 29811, tmp_path=None, expect_fail: bool = False, timeout: int = 240):
    script = os.path.join(str(tmp_path), "worker.py")
    with open(script, "w") as f:
        f.write(PRELUDE % {"root": ROOT} + textwrap.dedent(body))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(port), script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=dict(os.environ, OMP_NUM_THREADS="2"))
    if expect_fail:
        return r
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[7:])


def test_collectives_and_send_recv(tmp_path):
    res = run_ranks('''
        t = lt.Tensor(torch.tensor([1.0 + rank, 2.0]))
        pg.all_reduce(t)
        s = _unwrap(t).tolist()
        a = lt.Tensor(torch.tensor([1.0 + rank, 2.0])); pg.all_reduce(a, average=True)
        b = lt.Tensor(torch.tensor([float(rank)] * 3)); pg.broadcast(b, 1)
        g = pg.all_gather(lt.Tensor(torch.tensor([float(rank), 10.0 + rank])))
        rs = pg.reduce_scatter(lt.Tensor(torch.arange(4.0) * (rank + 1)))
        if rank == 0:
            pg.send_tensor(lt.Tensor(torch.arange(6.0).view(2, 3)), 1); got = None
        else:
            got = _unwrap(pg.recv_tensor(0)).tolist()
        shapes = [None]
        dist.broadcast_object_list(shapes if rank == 0 else shapes, 0)
        out = [None, None]
        dist.all_gather_object(out, (got, _unwrap(rs).tolist()))
        grads = [torch.full((5,), float(rank + 1)), torch.full((3,), 2.0 * (rank + 1))]
        lt.distributed.all_reduce_bucketed(grads, bucket_bytes=16, average=True)
        done(sum=s, avg=_unwrap(a).tolist(), bcast=_unwrap(b).tolist(), gather=_unwrap(g).tolist(), recv=out[1][0],
             rs0=out[0][1], rs1=out[1][1], bucket=[grads[0][0].item(), grads[1][0].item()], ws=pg.get_world_size())
    ''', tmp_path=tmp_path)
    assert res["sum"] == [3.0, 4.0] and res["avg"] == [1.5, 2.0] and res["bcast"] == [1.0, 1.0, 1.0]
    assert res["gather"] == [0.0, 10.0, 1.0, 11.0] and res["recv"] == [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]]
    assert res["rs0"] == [0.0, 3.0] and res["rs1"] == [6.0, 9.0] and res["bucket"] == [1.5, 3.0] and res["ws"] == 2


def test_tensor_and_sequence_parallel_match_full_linear(tmp_path):
    res = run_ranks('''
        from litetorch_b200.parallel.tp import _init_full
        torch.manual_seed(0)
        x = torch.randn(6, 2, 8)                                     # [T, B, in]
        col = lt.nn.ColumnParallelLinear(8, 12, True, gather_output=False)
        row = lt.nn.RowParallelLinear(12, 8, True, input_is_parallel=True)
        xin = x.clone().requires_grad_(True)
        y = row(lt.Ops.gelu(col(lt.Tensor(xin))))
        lt.Ops.sum(lt.Ops.mul(y, y)).backward()
        # single-process oracle with the full weights
        W1 = _init_full(12, 8); b1 = torch.empty(12).uniform_(-1 / math.sqrt(8), 1 / math.sqrt(8), generator=torch.Generator().manual_seed(4321))
        W2 = _init_full(8, 12, 1)
        xr = x.clone().requires_grad_(True)
        yr = torch.nn.functional.gelu(xr @ W1.t() + b1, approximate="tanh") @ W2.t()
        (yr * yr).sum().backward()
        e_fwd = float((_unwrap(y) - yr).abs().max()); e_dx = float((xin.grad - xr.grad).abs().max())
        # sequence parallel: activations sharded on dim 0 between the two layers' outsides
        col_sp = lt.nn.ColumnParallelLinear(8, 12, True, gather_output=False, sequence_parallel=True)
        row_sp = lt.nn.RowParallelLinear(12, 8, False, input_is_parallel=True, sequence_parallel=True)
        xs = x.chunk(world, 0)[rank].clone().requires_grad_(True)
        ys = row_sp(lt.Ops.gelu(col_sp(lt.Tensor(xs))))
        lt.Ops.sum(lt.Ops.mul(ys, ys)).backward()
        e_sp = float((_unwrap(ys) - yr.detach().chunk(world, 0)[rank]).abs().max())
        e_sp_dx = float((xs.grad - xr.grad.chunk(world, 0)[rank]).abs().max())
        # reference default behaviour: gathered output / full input
        full = lt.nn.ColumnParallelLinear(8, 12, True)(lt.Tensor(x))
        e_gather = float((_unwrap(full) - (x @ W1.t() + b1)).abs().max())
        errs = torch.tensor([e_fwd, e_dx, e_sp, e_sp_dx, e_gather]); dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        # vocab-parallel cross-entropy
        logits = torch.randn(10, 16, generator=torch.Generator().manual_seed(5)); tgt = torch.arange(10) % 16; tgt[0] = -100
        loc = logits[:, rank * 8:(rank + 1) * 8].clone().requires_grad_(True)
        l = lt.distributed.vocab_parallel_cross_entropy(loc, tgt, rank * 8)
        l.backward()
        lr = logits.clone().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(lr, tgt, ignore_index=-100); ref.backward()
        e_ce = torch.tensor([abs(float(l) - float(ref)), float((loc.grad - lr.grad[:, rank * 8:(rank + 1) * 8]).abs().max())])
        dist.all_reduce(e_ce, op=dist.ReduceOp.MAX)
        done(errs=errs.tolist(), ce=e_ce.tolist())
    ''', tmp_path=tmp_path, port=29821)
    assert max(res["errs"]) < 1e-5 and max(res["ce"]) < 1e-5, res


def test_pipeline_1f1b_matches_single_process(tmp_path):
    res = run_ranks('''
        torch.manual_seed(0)
        l1, l2 = lt.nn.Linear(4, 8), lt.nn.Linear(8, 2)             # same seed on both ranks -> identical weights
        class Stage(lt.nn.Module):
            def __init__(s, lin, act):
                super().__init__(); s.lin, s.act = lin, act
            def forward(s, x):
                y = s.lin(x)
                return lt.Ops.tanh(y) if s.act else y
        mbs = [lt.Tensor(torch.randn(3, 4, generator=torch.Generator().manual_seed(10 + i))) for i in range(4)]
        tg = [lt.Tensor(torch.randn(3, 2, generator=torch.Generator().manual_seed(50 + i))) for i in range(4)]
        stage = Stage(l1, True) if rank == 0 else Stage(l2, False)
        pp = lt.distributed.PipelineParallelModule(stage)
        loss = pp.train_step_1f1b(mbs, lambda out, t: lt.Ops.mse_loss(out, t), targets=tg)
        # oracle: whole model on every rank
        torch.manual_seed(0)
        r1, r2 = lt.nn.Linear(4, 8), lt.nn.Linear(8, 2)
        tot = 0.0
        for x, t in zip(mbs, tg):
            lo = lt.Ops.mse_loss(r2(lt.Ops.tanh(r1(x))), t); tot += lo.item()
            _unwrap(lo).div(4).backward()
        mine, ref = (l1, r1) if rank == 0 else (l2, r2)
        err = torch.tensor([float((_unwrap(mine.weight).grad - _unwrap(ref.weight).grad).abs().max())])
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        losses = [None, None]; dist.all_gather_object(losses, loss)
        fwd = pp.forward(mbs[0] if rank == 0 else None)
        done(err=err.item(), loss=losses[1], ref=tot / 4, fwd_shape=None)
    ''', tmp_path=tmp_path, port=29831)
    assert res["err"] < 1e-6 and abs(res["loss"] - res["ref"]) < 1e-6


def test_pipeline_1f1b_posts_receives_before_the_compute_they_overlap(tmp_path):
    """Order of events on the first of two stages in the 1F1B steady state: with overlap the receive of the gradient
    is posted before the forward that it runs under (R F B R F B ...); the grouped mode posts it after the forward.
    Both modes give the same gradients."""
    res = run_ranks('''
        import torch.distributed as tdist
        def run(overlap):
            torch.manual_seed(0)
            l1, l2 = lt.nn.Linear(4, 8), lt.nn.Linear(8, 2)
            log = []
            class Stage(lt.nn.Module):
                def __init__(s, lin):
                    super().__init__(); s.lin = lin
                def forward(s, x):
                    log.append("F"); return s.lin(x)
            mbs = [lt.Tensor(torch.randn(3, 4, generator=torch.Generator().manual_seed(10 + i))) for i in range(4)]
            tg = [lt.Tensor(torch.randn(3, 2, generator=torch.Generator().manual_seed(50 + i))) for i in range(4)]
            pp = lt.distributed.PipelineParallelModule(Stage(l1 if rank == 0 else l2))
            pp.overlap = overlap
            orig_irecv, orig_batch = tdist.irecv, tdist.batch_isend_irecv
            def irecv(*a, **k):
                log.append("R"); return orig_irecv(*a, **k)
            def batch(ops):
                if any(o.op is orig_irecv or o.op is irecv for o in ops): log.append("R")
                return orig_batch(ops)
            if overlap:
                tdist.irecv = irecv
            else:
                tdist.batch_isend_irecv = batch
            try:
                pp.train_step_1f1b(mbs, lambda out, t: lt.Ops.mse_loss(out, t), targets=tg)
            finally:
                tdist.irecv, tdist.batch_isend_irecv = orig_irecv, orig_batch
            g = _unwrap((l1 if rank == 0 else l2).weight).grad.clone()
            return "".join(log), g
        log_o, g_o = run(True)
        log_g, g_g = run(False)
        err = torch.tensor([float((g_o - g_g).abs().max())]); dist.all_reduce(err, op=dist.ReduceOp.MAX)
        done(overlapped=log_o, grouped=log_g, err=err.item())
    ''', tmp_path=tmp_path, port=29835)
    assert res["err"] < 1e-7
    # stage 0 of 2 with 4 micro-batches: one warm-up forward, three steady iterations, one drain backward
    assert res["overlapped"] == "F" + "RF" * 3 + "R", res
    assert res["grouped"] == "F" + "FR" * 3 + "R", res


def test_ring_attention_zigzag_and_moe_expert_parallel(tmp_path):
    res = run_ranks('''
        from litetorch_b200.parallel.cp import zigzag_split, zigzag_merge
        torch.manual_seed(0)
        B, H, Hkv, T, D = 1, 4, 2, 16, 8
        q, k, v = torch.randn(B, H, T, D), torch.randn(B, Hkv, T, D), torch.randn(B, Hkv, T, D)
        def full(causal):
            qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
            ke, ve = kk.repeat_interleave(2, 1), vv.repeat_interleave(2, 1)
            s = qq @ ke.transpose(-1, -2) / math.sqrt(D)
            if causal:
                s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            o = torch.softmax(s, -1) @ ve
            (o * o).sum().backward()
            return o.detach(), qq.grad, kk.grad, vv.grad
        errs = []
        for causal, zig in [(False, False), (True, False), (True, True)]:
            sp = (lambda t: zigzag_split(t, rank, world, 2)) if zig else (lambda t: t.chunk(world, 2)[rank].contiguous())
            ql, kl, vl = (sp(t).clone().requires_grad_(True) for t in (q, k, v))
            o = lt.distributed.ring_attention(ql, kl, vl, dist.group.WORLD, causal=causal, zigzag=zig)
            (o * o).sum().backward()
            oref, dq, dk, dv = full(causal)
            errs += [float((o.detach() - sp(oref)).abs().max()), float((ql.grad - sp(dq)).abs().max()),
                     float((kl.grad - sp(dk)).abs().max()), float((vl.grad - sp(dv)).abs().max())]
        parts = [None, None]; dist.all_gather_object(parts, zigzag_split(q, rank, world, 2))
        errs.append(float((zigzag_merge(parts, 2) - q).abs().max()))
        e = torch.tensor(errs); dist.all_reduce(e, op=dist.ReduceOp.MAX)
        # ---- MoE: expert parallel over 2 ranks vs all experts in one process
        xs = torch.randn(12, 8, generator=torch.Generator().manual_seed(3 + rank)).requires_grad_(True)
        moe = lt.distributed.MoEFeedForward(8, 16, 4, top_k=2, capacity_factor=8.0, group=dist.group.WORLD, seed=1)
        y = _unwrap(moe(lt.Tensor(xs)))
        (y * y).sum().backward()
        one = lt.distributed.MoEFeedForward.__new__(lt.distributed.MoEFeedForward)
        g = torch.Generator().manual_seed(1)
        gate = torch.empty(4, 8).normal_(0, 0.02, generator=g); wgu = torch.empty(4, 32, 8).normal_(0, 0.02, generator=g)
        wdn = torch.empty(4, 8, 16).normal_(0, 0.02, generator=g)
        xr = xs.detach().clone().requires_grad_(True)
        p = torch.softmax(xr @ gate.t(), -1); tp_, ti = p.topk(2, -1); tw = tp_ / tp_.sum(-1, keepdim=True)
        yr = torch.zeros_like(xr)
        for n in range(12):
            for j in range(2):
                e_ = int(ti[n, j]); gu = xr[n] @ wgu[e_].t()
                yr[n] = yr[n] + tw[n, j] * ((torch.nn.functional.silu(gu[:16]) * gu[16:]) @ wdn[e_].t())
        (yr * yr).sum().backward()
        em = torch.tensor([float((y - yr).abs().max()), float((xs.grad - xr.grad).abs().max())]); dist.all_reduce(em, op=dist.ReduceOp.MAX)
        tight = lt.distributed.MoEFeedForward(8, 16, 4, top_k=2, capacity_factor=0.5, group=dist.group.WORLD, seed=1)
        tight(lt.Tensor(xs.detach()))
        done(ring=e.tolist(), moe=em.tolist(), dropped=tight.last_dropped, aux=float(moe.last_aux_loss))
    ''', tmp_path=tmp_path, port=29841)
    assert max(res["ring"]) < 1e-4, res
    assert max(res["moe"]) < 1e-5 and res["dropped"] > 0 and 0.005 < res["aux"] < 0.05, res


def test_fsdp_wrappers_zero3_dtensor_mesh(tmp_path):
    res = run_ranks('''
        torch.manual_seed(0)
        net = lt.nn.Sequential([lt.nn.Linear(5, 7), lt.nn.Tanh(), lt.nn.Linear(7, 3)])
        ref = [_unwrap(p).detach().clone() for p in net.parameters()]
        x = torch.randn(4, 5, generator=torch.Generator().manual_seed(20 + rank))
        f = lt.distributed.FullyShardedDataParallel(net)
        shard_sizes = [_unwrap(p.shard).numel() for p in f.parameters()]
        emptied = all(list(_unwrap(p).shape) == [_unwrap(p.shard).numel()] for p in f.parameters())
        out = f(lt.Tensor(x))
        lt.Ops.sum(lt.Ops.mul(out, out)).backward()
        f.shard_parameters()
        opt = lt.optim.ZeRO3Optimizer(f.parameters(), lr=0.1, weight_decay=0.0)
        opt.step()
        f.gather_parameters()
        new = [_unwrap(p).detach().clone() for p in f.parameters()]
        # oracle: replicated model, summed grads, same Adam
        ws = [r.clone().requires_grad_(True) for r in ref]
        tot = 0
        xs = [torch.randn(4, 5, generator=torch.Generator().manual_seed(20 + r)) for r in range(world)]
        for xx in xs:
            o = torch.tanh(xx @ ws[0].t() + ws[1]) @ ws[2].t() + ws[3]; tot = tot + (o * o).sum()
        tot.backward()
        o2 = torch.optim.AdamW(ws, lr=0.1, weight_decay=0.0); o2.step()
        err = max(float((a - b.detach()).abs().max()) for a, b in zip(new, ws))
        # hook-based fully_shard
        torch.manual_seed(0)
        net2 = lt.distributed.FSDP.fully_shard(lt.nn.Sequential([lt.nn.Linear(5, 7), lt.nn.Tanh(), lt.nn.Linear(7, 3)]))
        o = net2(lt.Tensor(x)); lt.Ops.sum(lt.Ops.mul(o, o)).backward()
        sg = [_unwrap(s).grad for s in lt.distributed.FSDP.shards(net2)]
        full_g = ws[0].grad.reshape(-1); per = (full_g.numel() + world - 1) // world
        pad = torch.zeros(per * world); pad[:full_g.numel()] = full_g
        err2 = float((sg[0] - pad[rank * per:(rank + 1) * per]).abs().max())
        # mesh + DTensor
        mesh = lt.distributed.DeviceMesh([1, 2], "dp tp")
        P = lt.distributed.Placement
        base = torch.arange(8.0).view(2, 4)
        d = lt.distributed.distribute_tensor(lt.Tensor(base), mesh, [P.replicate(), P.shard(1)])
        local = _unwrap(d.to_local()).tolist()
        back = _unwrap(d.full_tensor()).tolist()
        part = lt.distributed.DTensor(lt.Tensor(torch.ones(2) * (rank + 1)), mesh, [P.replicate(), P.partial()])
        red = _unwrap(part.redistribute([P.replicate(), P.replicate()]).to_local()).tolist()
        e = torch.tensor([err, err2]); dist.all_reduce(e, op=dist.ReduceOp.MAX)
        done(err=e.tolist(), shard_sizes=shard_sizes, emptied=emptied, local=local, back=back, red=red,
             coord=mesh.get_coordinate(), tp_ranks=mesh.ranks_along("tp"))
    ''', tmp_path=tmp_path, port=29851)
    assert max(res["err"]) < 1e-5, res
    assert res["shard_sizes"] == [18, 4, 11, 2] and res["emptied"]
    assert res["local"] == [[0.0, 1.0], [4.0, 5.0]] and res["back"] == [[0, 1, 2, 3], [4, 5, 6, 7]] and res["red"] == [3.0, 3.0]
    assert res["coord"] == [0, 0] and res["tp_ranks"] == [0, 1]


def test_rank_that_leaves_is_detected_not_hung(tmp_path):
    """Rank 1 exits between steps; rank 0 learns it from the heartbeat store before its next collective and from the
    short process-group timeout when it tries one anyway."""
    r = run_ranks('''
        import time
        from litetorch_b200.parallel.process_group import TCPStore, Watchdog, RankFailure
        store = TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 7, is_server=(rank == 0))
        wd = Watchdog(store, rank, interval_s=0.05, ttl_s=0.5)
        t = lt.Tensor(torch.ones(2)); pg.all_reduce(t)                # step 1 works
        store.barrier("warm", world, 10.0)
        if rank == 1:
            wd.stop(); store.close(); os._exit(0)                     # leaves with nothing in flight
        time.sleep(1.2)
        try:
            wd.check(); print("RESULT " + json.dumps({"detected": False}))
        except RankFailure as e:
            print("RESULT " + json.dumps({"detected": True, "msg": str(e)}))
        try:
            store.barrier("after", world, 0.3); print("BARRIER ok")
        except TimeoutError:
            print("BARRIER timeout")
        sys.stdout.flush()
        os._exit(0)
    ''', tmp_path=tmp_path, port=29861, expect_fail=True, timeout=120)
    assert 'RESULT {"detected": true' in r.stdout and "[1]" in r.stdout and "BARRIER timeout" in r.stdout, r.stdout + r.stderr[-1500:]


def test_reference_environment_variables_are_honoured(tmp_path):
    """LITETORCH_RENDEZVOUS_FILE selects the file rendezvous (the reference publishes its communicator id through that
    file), the 128-byte id travels through `<file>.ncclid` for the native NCCL bridge, LITETORCH_NO_GPU switches the GPU
    off and LITETORCH_NUM_THREADS sizes the host thread pool."""
    rend = os.path.join(str(tmp_path), "rendezvous")
    script = os.path.join(str(tmp_path), "w.py")
    with open(script, "w") as f:
        f.write(textwrap.dedent('''
            import json, os, sys, torch
            sys.path.insert(0, %r)
            import torch.distributed as dist
            import litetorch_b200 as lt
            from litetorch_b200.core import _unwrap
            from litetorch_b200.parallel import nccl_native as NN
            rank = int(sys.argv[1])
            # a port nobody listens on: only the file rendezvous can bring the two ranks together
            pg = lt.distributed.init_process_group(rank, 2, "127.0.0.1", 1, backend="gloo", timeout_s=60)
            t = lt.Tensor(torch.tensor([1.0 + rank]))
            pg.all_reduce(t)
            path = NN._id_file()
            if rank == 0:
                NN.publish_id_file(path, bytes(range(128)))
            raw = NN.read_id_file(path, 30)
            import ctypes
            from litetorch_b200._native import host_lib
            L = host_lib(); L.lt_pool_threads.restype = ctypes.c_int
            print("RESULT " + json.dumps({"sum": _unwrap(t).item(), "id_ok": raw == bytes(range(128)), "gpu": lt.is_gpu_available(),
                                          "dev": str(lt.auto_device()), "backend": lt.get_backend_name(), "threads": L.lt_pool_threads()}))
            dist.barrier(); pg.shutdown()
        ''' % ROOT))
    env = dict(os.environ, LITETORCH_RENDEZVOUS_FILE=rend, LITETORCH_NO_GPU="1", LITETORCH_NUM_THREADS="3", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, script, str(r)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
             for r in range(2)]
    outs = [p.communicate(timeout=240) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, o[-1500:] + e[-3000:]
    for o, _ in outs:
        res = json.loads([l for l in o.splitlines() if l.startswith("RESULT ")][-1][7:])
        assert res["sum"] == 3.0 and res["id_ok"] and res["gpu"] is False and res["backend"] == "CPU" and res["threads"] == 3
        assert "cpu" in res["dev"].lower()
    from litetorch_b200.parallel import nccl_native as NN
    with pytest.raises(NN.NcclError):
        NN.read_id_file(os.path.join(str(tmp_path), "never_written"), 0.2)


def test_reference_distributed_test_replay(tmp_path):
    """The expectations of the reference's tests/distributed_test.cpp through the module-level functions: its host
    all-reduce averages (here `average=True`), `recv_tensor` gives the destination the sender's shape, and a two-stage
    pipeline of doubling modules turns 5 into 20 on the last rank."""
    res = run_ranks('''
        D = lt.distributed
        cpu = lt.Device("cpu")
        t = lt.Tensor.from_vector([float(rank), float(rank * 2)], [2], cpu, False)
        D.all_reduce(t, average=True)
        bc = lt.Tensor.from_vector([42.0 if rank == 0 else 0.0], [1], cpu, False)
        D.broadcast(bc, 0)
        got = None
        if rank == 0:
            D.send_tensor(lt.Tensor.from_vector([100.0, 200.0, 300.0], [3], cpu, False), 1)
        else:
            r = lt.Tensor.create([1], cpu)
            D.recv_tensor(r, 0)
            got = [r.shape, r.to_vector()]
        class TimesTwo(lt.nn.Module):
            def forward(self, input):
                return lt.Ops.mul(input, lt.Tensor.from_vector([2.0], [1], cpu, False))
        pp = D.PipelineParallelModule(TimesTwo())
        out = pp.forward(lt.Tensor.from_vector([5.0], [1], cpu, False) if rank == 0 else None)
        last = out.to_vector() if rank == 1 else None
        sh = lt.Tensor.from_vector([0.0, 0.0], [2], cpu, False)
        D.reduce_scatter(sh, lt.Tensor.from_vector([1.0, 2.0, 3.0, 4.0], [4], cpu, False))
        h = D.all_reduce_async(lt.Tensor.from_vector([1.0], [1], cpu, False)); h.wait()
        objs = [None, None]
        dist.all_gather_object(objs, (got, last, sh.to_vector()))
        if rank == 0:
            print("RESULT " + json.dumps(dict(avg=t.to_vector(), bc=bc.to_vector(), recv=objs[1][0], last=objs[1][1],
                                              rs=[objs[0][2], objs[1][2]], ids=[D.get_rank(), D.get_world_size()])))
        D.barrier()
        D.shutdown()
    ''', tmp_path=tmp_path, port=29877)
    assert res["avg"] == [0.5, 1.0] and res["bc"] == [42.0]
    assert res["recv"] == [[3], [100.0, 200.0, 300.0]] and res["last"] == [20.0]
    assert res["rs"] == [[2.0, 4.0], [6.0, 8.0]] and res["ids"] == [0, 2]

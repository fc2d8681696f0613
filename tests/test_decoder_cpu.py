"""The parallel decoder (tensor + sequence parallel, context parallel ring attention, expert parallel MoE, pipeline
stages) on CPU gloo ranks: the sharded model reproduces the loss and the gradients of the same model on one rank,
and the three benchmark layouts run end to end on small shapes."""
import json
import os
import subprocess
import sys

import pytest

from test_distributed_cpu import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tp_sp_and_cp_match_single_rank(tmp_path):
    res = run_ranks('''
        from litetorch_b200.models.decoder import PRESETS, ParallelDecoder, ParallelDims, shard_batch
        cfg = PRESETS["tiny-dense"]
        torch.manual_seed(0)
        ids = torch.randint(0, cfg.vocab, (2, 129))
        x, y = ids[:, :-1], ids[:, 1:]
        out = {}
        for mode in ("tp", "cp", "ulysses"):
            grp = dist.group.WORLD
            dims = ParallelDims(tp=grp if mode == "tp" else None, cp=grp if mode != "tp" else None, zigzag=True,
                                cp_mode="ulysses" if mode == "ulysses" else "ring")
            m = ParallelDecoder(cfg, dims, device="cpu", dtype=torch.float32, seed=3)
            loss = m.forward_loss(shard_batch(x, dims), shard_batch(y, dims))
            loss.backward()
            m.reduce_gradients()
            # the same weights on one rank: gather the tensor-parallel shards
            ref = ParallelDecoder(cfg, ParallelDims(), device="cpu", dtype=torch.float32, seed=3)
            def gather(t, dim):
                parts = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(parts, t.detach().contiguous())
                return parts if dim is None else torch.cat(parts, dim)
            with torch.no_grad():
                if mode == "tp":
                    D = cfg.head_dim
                    for b, rb in zip(m.blocks, ref.blocks):
                        parts = gather(b.wqkv, None)
                        q = torch.cat([p[:b.hq * D] for p in parts]); k = torch.cat([p[b.hq * D:(b.hq + b.hkv) * D] for p in parts])
                        v = torch.cat([p[(b.hq + b.hkv) * D:] for p in parts])
                        rb.wqkv.copy_(torch.cat([q, k, v]))
                        rb.wo.copy_(gather(b.wo, 1))
                        F = cfg.ffn // world
                        gu = gather(b.w_gu, None)
                        rb.w_gu.copy_(torch.cat([torch.cat([p[:F] for p in gu]), torch.cat([p[F:] for p in gu])]))
                        rb.w_dn.copy_(gather(b.w_dn, 1))
                    ref.head.copy_(gather(m.head, 0))
                    ref.embed.copy_(m.embed)
                else:
                    for p, rp in zip(m.parameters(), ref.parameters()):
                        rp.copy_(p)
            ref_loss = ref.forward_loss(x, y)
            ref_loss.backward()
            lv = loss.detach().clone()
            if mode != "tp":
                dist.all_reduce(lv); lv /= world       # every rank holds the mean over its own tokens
            # gradients of replicated parameters must agree with the single-rank model
            g_err = max(float((a.grad - b.grad).abs().max() / (b.grad.abs().max() + 1e-12))
                        for a, b in [(m.embed, ref.embed), (m.blocks[0].norm1, ref.blocks[0].norm1),
                                     (m.blocks[1].norm2, ref.blocks[1].norm2), (m.final_norm, ref.final_norm)])
            if mode != "tp":
                g_err = max(g_err, float((m.blocks[0].wqkv.grad - ref.blocks[0].wqkv.grad).abs().max()
                                         / ref.blocks[0].wqkv.grad.abs().max()))
            else:
                F = cfg.ffn // world
                mine = ref.blocks[1].w_dn.grad[:, rank * F:(rank + 1) * F]
                g_err = max(g_err, float((m.blocks[1].w_dn.grad - mine).abs().max() / mine.abs().max()))
            out[mode] = [float(lv), float(ref_loss), g_err]
        done(**out)
    ''', nproc=2, port=29841, tmp_path=tmp_path, timeout=600)
    for mode in ("tp", "cp", "ulysses"):
        loss, ref, g_err = res[mode]
        assert abs(loss - ref) < 2e-4 * abs(ref), (mode, loss, ref)
        assert g_err < 2e-3, (mode, g_err)


@pytest.mark.parametrize("config,nproc,extra", [("tp8", 2, []), ("ep8", 2, []), ("hybrid", 8, ["--seq", "256"])])
def test_benchmark_layouts_run_on_small_shapes(config, nproc, extra):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(29850 + nproc), "-m", "litetorch_b200.models.run_config", "--config", config,
           "--tiny", "--steps", "2", "--warmup", "1"] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    d = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert d["n_gpus"] == nproc and d["tokens_per_s"] > 0
    assert 4.0 < d["loss"] < 8.0          # ln(512) = 6.24 at initialisation


def test_tp2_x_cp2_on_four_ranks_matches_single_rank(tmp_path):
    """Tensor + sequence parallelism inside context parallelism (the two inner axes of the hybrid layout): loss and
    gradients of sharded and replicated parameters equal the single-rank model."""
    res = run_ranks('''
        from litetorch_b200.models.decoder import PRESETS, ParallelDecoder, ParallelDims, shard_batch
        from litetorch_b200.models.run_config import _make_groups
        cfg = PRESETS["tiny-dense"]
        torch.manual_seed(0)
        ids = torch.randint(0, cfg.vocab, (2, 129))
        x, y = ids[:, :-1], ids[:, 1:]
        groups, _ = _make_groups(world, rank, 2, 2, 1, 1)
        dims = ParallelDims(tp=groups["tp"], cp=groups["cp"], zigzag=True)
        m = ParallelDecoder(cfg, dims, device="cpu", dtype=torch.float32, seed=3)
        loss = m.forward_loss(shard_batch(x, dims), shard_batch(y, dims))
        loss.backward()
        m.reduce_gradients()
        ref = ParallelDecoder(cfg, ParallelDims(), device="cpu", dtype=torch.float32, seed=3)
        tpw = 2
        def gather(t, dim):
            parts = [torch.empty_like(t) for _ in range(tpw)]
            dist.all_gather(parts, t.detach().contiguous(), group=groups["tp"])
            return parts if dim is None else torch.cat(parts, dim)
        with torch.no_grad():
            D = cfg.head_dim
            for b, rb in zip(m.blocks, ref.blocks):
                parts = gather(b.wqkv, None)
                q = torch.cat([p[:b.hq * D] for p in parts]); k = torch.cat([p[b.hq * D:(b.hq + b.hkv) * D] for p in parts])
                v = torch.cat([p[(b.hq + b.hkv) * D:] for p in parts])
                rb.wqkv.copy_(torch.cat([q, k, v]))
                rb.wo.copy_(gather(b.wo, 1))
                F = cfg.ffn // tpw
                gu = gather(b.w_gu, None)
                rb.w_gu.copy_(torch.cat([torch.cat([p[:F] for p in gu]), torch.cat([p[F:] for p in gu])]))
                rb.w_dn.copy_(gather(b.w_dn, 1))
            ref.head.copy_(gather(m.head, 0))
            ref.embed.copy_(m.embed)
        ref_loss = ref.forward_loss(x, y)
        ref_loss.backward()
        lv = loss.detach().clone()
        dist.all_reduce(lv, group=groups["cp"]); lv /= 2      # every context-parallel rank holds the mean over its tokens
        g_err = max(float((a.grad - b.grad).abs().max() / (b.grad.abs().max() + 1e-12))
                    for a, b in [(m.embed, ref.embed), (m.blocks[0].norm1, ref.blocks[0].norm1),
                                 (m.blocks[1].norm2, ref.blocks[1].norm2), (m.final_norm, ref.final_norm)])
        F = cfg.ffn // tpw
        tr = dist.get_rank(groups["tp"])
        mine = ref.blocks[1].w_dn.grad[:, tr * F:(tr + 1) * F]
        g_err = max(g_err, float((m.blocks[1].w_dn.grad - mine).abs().max() / mine.abs().max()))
        done(loss=float(lv), ref=float(ref_loss), g_err=g_err)
    ''', nproc=4, port=29861, tmp_path=tmp_path, timeout=600)
    assert abs(res["loss"] - res["ref"]) < 2e-4 * abs(res["ref"]), res
    assert res["g_err"] < 2e-3, res


def test_parallel_layouts_follow_the_single_rank_loss_curve():
    """Three optimisation steps of the tiny hybrid model: context parallel x pipeline parallel on four ranks ends on the
    same loss as one rank (same data, same initial weights; the reported loss is the global mean)."""
    def run(layout, nproc, port):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
               "127.0.0.1", "--master-port", str(port), "-m", "litetorch_b200.models.run_config", "--config", "hybrid", "--tiny",
               "--steps", "2", "--warmup", "1", "--layout", layout, "--micro", "1", "--seq", "256"]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env=dict(os.environ, OMP_NUM_THREADS="1"))
        assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
        return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])["loss"]
    one = run("1,1,1", 1, 29871)
    four = run("1,2,2", 4, 29872)
    assert abs(one - four) < 2e-4, (one, four)
    # weights are drawn unit by unit, so tensor parallelism starts from the same model too: the full 4D layout
    # (TP2 x CP2 x PP2 on eight ranks) follows the same curve
    eight = run("2,2,2", 8, 29873)
    assert abs(one - eight) < 5e-4, (one, eight)

"""Ulysses sequence-parallel attention on gloo ranks: output and gradients equal full attention on one rank."""
from test_distributed_cpu import run_ranks


def test_ulysses_matches_full_attention(tmp_path):
    res = run_ranks('''
        import math
        from litetorch_b200.parallel.ulysses import ulysses_attention, seq_to_head, head_to_seq
        worst = 0.0
        for (Hq, Hkv) in [(4, 2), (4, 1)]:
            B, T, D = 2, 32, 16
            g = torch.Generator().manual_seed(5)
            q, k, v, do = (torch.randn(B, T, h, D, generator=g) for h in (Hq, Hkv, Hkv, Hq))
            sp = lambda t: t.chunk(world, 1)[rank].contiguous()
            ql, kl, vl = (sp(t).clone().requires_grad_(True) for t in (q, k, v))
            o = ulysses_attention(ql, kl, vl, dist.group.WORLD, causal=True)
            o.backward(sp(do))
            qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
            G = Hq // Hkv
            s = torch.einsum("bthd,bshd->bhts", qf, kf.repeat_interleave(G, 2)) / math.sqrt(D)
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            of = torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), vf.repeat_interleave(G, 2))
            of.backward(do)
            for a, b in ((o, sp(of.detach())), (ql.grad, sp(qf.grad)), (kl.grad, sp(kf.grad)), (vl.grad, sp(vf.grad))):
                worst = max(worst, float((a - b).abs().max()))
        x = torch.arange(2 * 4 * 4 * 3, dtype=torch.float32).view(2, 4, 4, 3) + 1000 * rank
        back = head_to_seq(seq_to_head(x, dist.group.WORLD), dist.group.WORLD)
        done(worst=worst, roundtrip=bool(torch.equal(back, x)))
    ''', tmp_path=tmp_path, port=29823)
    assert res["worst"] < 1e-4 and res["roundtrip"], res

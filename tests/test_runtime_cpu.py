"""Native host runtime on CPU: checkpoint formats, data loader, JIT, serving scheduler, allocator, stores."""
import os
import struct
import threading
import time
import zlib

import pytest
import torch

import litetorch_b200 as lt
from litetorch_b200.core import _unwrap


# ------------------------------------------------------------------ checkpoints
def test_ltw1_layout_crc_and_roundtrip(tmp_path):
    net = lt.nn.Sequential([lt.nn.Linear(3, 2), lt.nn.LayerNorm([2])])
    path = str(tmp_path / "m.ltw1")
    lt.save(net, path)
    raw = open(path, "rb").read()
    assert raw[:4] == b"LTW1" and struct.unpack("<I", raw[4:8])[0] == 4
    ndims, d0, d1, numel = struct.unpack("<Iqq Q".replace(" ", ""), raw[8:8 + 4 + 16 + 8])
    assert (ndims, d0, d1, numel) == (2, 2, 3, 6)
    assert struct.unpack("<I", raw[-4:])[0] == zlib.crc32(raw[:-4])           # CRC-32/IEEE over everything before it
    assert len(raw) == 4 + 4 + (4 + 16 + 8 + 24) + (4 + 8 + 8 + 8) * 3 + 4
    other = lt.nn.Sequential([lt.nn.Linear(3, 2), lt.nn.LayerNorm([2])])
    lt.load(other, path)
    for a, b in zip(net.parameters(), other.parameters()):
        assert torch.equal(_unwrap(a), _unwrap(b))


def test_crc32_equals_zlib_at_every_alignment_and_tail_length():
    import ctypes
    from litetorch_b200._native import host_lib
    lib = host_lib()
    lib.lt_crc32.restype = ctypes.c_uint32
    lib.lt_crc32.argtypes = [ctypes.c_char_p, ctypes.c_uint64]
    blob = bytes((i * 131 + 7) % 256 for i in range(4099))
    for n in list(range(0, 40)) + [255, 256, 257, 4096, 4099]:
        for off in (0, 1, 3):
            piece = blob[off:off + n]
            assert lib.lt_crc32(piece, len(piece)) == zlib.crc32(piece), (n, off)


def test_corrupt_or_mismatched_checkpoint_leaves_model_untouched(tmp_path):
    net = lt.nn.Linear(4, 4)
    path = str(tmp_path / "m.ltw1")
    lt.save_parameters(net.parameters(), path)
    raw = bytearray(open(path, "rb").read())
    raw[40] ^= 0xFF
    bad = str(tmp_path / "bad.ltw1")
    open(bad, "wb").write(raw)
    victim = lt.nn.Linear(4, 4)
    before = [_unwrap(p).clone() for p in victim.parameters()]
    with pytest.raises(lt.serialization.CheckpointError, match="CRC"):
        lt.load_parameters(victim.parameters(), bad)
    open(bad, "wb").write(bytes(raw[:30]))
    with pytest.raises(lt.serialization.CheckpointError):
        lt.load_parameters(victim.parameters(), bad)
    with pytest.raises(lt.serialization.CheckpointError, match="shape|tensors"):
        lt.load_parameters(lt.nn.Linear(4, 5).parameters(), path)
    assert all(torch.equal(_unwrap(p), b) for p, b in zip(victim.parameters(), before))


def test_a_save_that_dies_half_way_leaves_the_previous_file_intact(tmp_path):
    """The writer builds the file under a temporary name and renames it at the end: a process that exits in the middle
    of `lt.save` does not damage the file that was there, and a finished save leaves no temporary file behind."""
    import subprocess
    import sys
    net = lt.nn.Linear(4, 4)
    path = str(tmp_path / "m.ltw1")
    lt.save(net, path)
    good = open(path, "rb").read()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys, os; sys.path.insert(0, %r)\n"
            "import ctypes\n"
            "from litetorch_b200 import serialization as S\n"
            "lib = S._lib()\n"
            "w = lib.lt_ckpt_writer_open(%r.encode(), b'LTW1')\n"
            "lib.lt_ckpt_write_u32(w, 99)\n"
            "os._exit(0)\n") % (root, path)
    subprocess.run([sys.executable, "-c", code], check=True, timeout=120)
    assert open(path, "rb").read() == good
    lt.load(lt.nn.Linear(4, 4), path)
    lt.save(net, path)
    leftovers = [f for f in os.listdir(tmp_path) if f.startswith("m.ltw1.tmp.")]
    assert len(leftovers) == 1                      # only the dead process's partial file; the finished saves left none


@pytest.mark.parametrize("kind,magic", [("adam", b"LTAD"), ("adamw", b"LTAW"), ("sgd", b"LTSG"), ("rmsprop", b"LTRP")])
def test_optimizer_state_roundtrip_resumes_exactly(tmp_path, kind, magic):
    torch.manual_seed(0)
    mk = {"adam": lambda p: lt.optim.Adam(p, lr=1e-2), "adamw": lambda p: lt.optim.AdamW(p, lr=1e-2),
          "sgd": lambda p: lt.optim.SGD(p, lr=1e-2, momentum=0.9), "rmsprop": lambda p: lt.optim.RMSprop(p, lr=1e-2)}[kind]
    w = torch.randn(3, 3)
    grads = [torch.randn(3, 3) for _ in range(4)]
    a = lt.Tensor(w.clone().requires_grad_(True))
    oa = mk([a])
    for g in grads[:2]:
        _unwrap(a).grad = g.clone()
        oa.step()
    ck_o, ck_p = str(tmp_path / "o.bin"), str(tmp_path / "p.bin")
    lt.save(oa, ck_o)
    lt.save_parameters([a], ck_p)
    assert open(ck_o, "rb").read(4) == magic
    for g in grads[2:]:
        _unwrap(a).grad = g.clone()
        oa.step()
    b = lt.Tensor(torch.zeros(3, 3, requires_grad=True))
    ob = mk([b])
    lt.load_parameters([b], ck_p)
    lt.load(ob, ck_o)
    for g in grads[2:]:
        _unwrap(b).grad = g.clone()
        ob.step()
    assert torch.allclose(_unwrap(a), _unwrap(b), atol=1e-7)


def test_sharded_checkpoint_manifest(tmp_path):
    d = str(tmp_path / "ck")
    for r in range(2):
        lt.serialization.save_sharded(d, [torch.full((4,), float(r))], r, 2, meta={"step": 7})
    assert lt.serialization.load_sharded(d, 1, 2)[0].tolist() == [1.0] * 4
    with pytest.raises(lt.serialization.CheckpointError):
        lt.serialization.load_sharded(d, 0, 4)


# ------------------------------------------------------------------ data loader
def _loader(n=100, bs=16, shuffle=True, seed=3):
    x = lt.Tensor(torch.arange(n, dtype=torch.float32)[:, None].repeat(1, 2))
    y = lt.Tensor(torch.arange(n, dtype=torch.float32))
    return lt.data.DataLoader(lt.data.TensorDataset(x, y), bs, shuffle, lt.Device("cpu"), 2, seed=seed)


def test_dataloader_epoch_covers_dataset_and_reshuffles():
    dl = _loader()
    seen = []
    while True:
        b = dl.next()
        if b is None:
            break
        assert torch.equal(_unwrap(b[0])[:, 0], _unwrap(b[1]))
        seen += _unwrap(b[1]).tolist()
    assert sorted(seen) == list(range(100)) and seen != sorted(seen) and dl.next() is None
    dl.reset()
    second = [v for b in dl for v in _unwrap(b[1]).tolist()]
    assert sorted(second) == list(range(100)) and second != seen


def test_dataloader_large_batches_are_assembled_by_the_thread_pool():
    """Batches above about 1 MB are copied sample by sample on the host thread pool; rows must land in order."""
    n, w = 3000, 700
    x = torch.arange(n, dtype=torch.float32)[:, None] + torch.arange(w, dtype=torch.float32)[None] / 1024
    dl = lt.data.DataLoader(lt.data.TensorDataset(lt.Tensor(x), lt.Tensor(torch.arange(n, dtype=torch.float32))), 1024, True,
                            lt.Device("cpu"), 2, seed=5)
    rows = 0
    for bx, by in dl:
        bx, by = _unwrap(bx), _unwrap(by)
        assert torch.equal(bx, x[by.long()])
        rows += by.numel()
    assert rows == n


def test_dataloader_state_file_layout_and_deterministic_resume(tmp_path):
    dl = _loader()
    for _ in range(3):
        dl.next()
    path = str(tmp_path / "dl.bin")
    dl.save_state(path)
    raw = open(path, "rb").read()
    assert len(raw) == 4 + 8 * 3 + 1 + 8 + 100 * 8 + 4 and raw[:4] == b"LTDL"      # same size as the reference sample
    cur, wrk, ep = struct.unpack("<QQQ", raw[4:28])
    assert cur == 48 and raw[28] == 1 and struct.unpack("<Q", raw[29:37])[0] == 100
    assert struct.unpack("<I", raw[-4:])[0] == zlib.crc32(raw[:-4])
    rest = [v for b in dl for v in _unwrap(b[1]).tolist()]
    dl2 = _loader(seed=99)
    dl2.load_state(path)
    assert [v for b in dl2 for v in _unwrap(b[1]).tolist()] == rest
    open(path, "wb").write(raw[:-1] + b"\x00")
    with pytest.raises(RuntimeError, match="CRC"):
        dl2.load_state(path)


def test_token_stream_windows_ranks_epochs_and_exact_resume(tmp_path):
    import numpy as np
    path = str(tmp_path / "tokens.bin")
    n = 5000
    np.arange(n, dtype=np.uint32).tofile(path)                      # token i has the value i: windows are recognisable
    T, B, W = 16, 3, 2
    streams = [lt.data.TokenStream(path, T, B, dtype="uint32", shuffle=True, seed=5, rank=r, world=W) for r in range(W)]
    assert streams[0].num_tokens == n and streams[0].num_windows == (n - 1) // T
    per_epoch = streams[0].batches_per_epoch
    assert per_epoch == (streams[0].num_windows // W) // B
    seen = []
    for s in streams:
        mine = []
        while (b := s.next()) is not None:
            tok, tgt = b
            assert tok.shape == (B, T) and tok.dtype == torch.int64
            assert torch.equal(tgt, tok + 1) and bool((tok[:, 1:] == tok[:, :-1] + 1).all())
            assert bool((tok[:, 0] % T == 0).all())                  # window i starts at token i * T
            mine += (tok[:, 0] // T).tolist()
        assert s.next() is None and len(mine) == per_epoch * B       # the end of the epoch is sticky
        seen.append(mine)
    assert not set(seen[0]) & set(seen[1]) and len(set(seen[0])) == len(seen[0])   # ranks see disjoint windows, once
    first_epoch = list(seen[0])
    streams[0].next_epoch()
    second = []
    while (b := streams[0].next()) is not None:
        second += (b[0][:, 0] // T).tolist()
    assert streams[0].epoch == 1 and second != first_epoch           # a new permutation
    # exact resume: take some batches, save, read the rest; a fresh stream that loads the state reads the same rest
    a = lt.data.TokenStream(path, T, B, dtype="uint32", shuffle=True, seed=5, rank=1, world=W)
    a.next_epoch()
    for _ in range(7):
        a.next()
    a.save_state(str(tmp_path / "ts.json"))
    rest = []
    for _ in range(per_epoch + 5):                                   # across the epoch boundary
        b = a.next()
        if b is None:
            a.next_epoch()
            continue
        rest.append(b[0].clone())
    c = lt.data.TokenStream(path, T, B, dtype="uint32", shuffle=True, seed=5, rank=1, world=W)
    c.load_state(str(tmp_path / "ts.json"))
    assert (c.epoch, c.position) == (1, 7)
    again = []
    for _ in range(per_epoch + 5):
        b = c.next()
        if b is None:
            c.next_epoch()
            continue
        again.append(b[0].clone())
    assert len(again) == len(rest) and all(torch.equal(x, y) for x, y in zip(again, rest))
    with pytest.raises(RuntimeError):
        lt.data.TokenStream(path, T, B + 1, dtype="uint32", rank=1, world=W).load_state(str(tmp_path / "ts.json"))
    with pytest.raises(RuntimeError):
        lt.data.TokenStream(path, 4000, 4, dtype="uint32")           # not enough windows for one batch
    # sequential order without shuffling, 16-bit tokens, the endless iterator
    np.arange(300, dtype=np.uint16).tofile(str(tmp_path / "small.bin"))
    seq = lt.data.TokenStream(str(tmp_path / "small.bin"), 10, 2, shuffle=False)
    it = iter(seq)
    firsts = [next(it)[0][:, 0].tolist() for _ in range(seq.batches_per_epoch + 1)]
    assert firsts[0] == [0, 10] and firsts[1] == [20, 30] and firsts[-1] == [0, 10] and seq.epoch == 1


def test_pack_examples_masks_prompts_padding_and_example_boundaries():
    tok, tgt = lt.data.pack_examples([([1, 2, 3], [4, 5]), ([6], [7, 8, 9]), ([10, 11], [12])], seq_len=8, pad_id=0)
    assert tok.tolist() == [[1, 2, 3, 4, 5, 6, 7, 8], [10, 11, 12, 0, 0, 0, 0, 0]]
    assert tgt.tolist() == [[-100, -100, 4, 5, -100, 7, 8, 9], [-100, 12, -100, -100, -100, -100, -100, -100]]
    tok, tgt = lt.data.pack_examples([([1, 2], [3])], seq_len=4, mask_prompt=False)
    assert tgt.tolist() == [[2, 3, -100, -100]]
    tok, tgt = lt.data.pack_examples([(list(range(1, 8)), [8, 9, 10])], seq_len=4)          # longer than a row: cut
    assert tok.tolist() == [[1, 2, 3, 4]] and tgt.tolist() == [[-100] * 4]
    with pytest.raises(ValueError):
        lt.data.pack_examples([], seq_len=4)


def test_python_dataset_subclass():
    class Sq(lt.data.Dataset):
        def size(self): return 10
        def get(self, i): return lt.Tensor(torch.tensor([float(i)])), lt.Tensor(torch.tensor(float(i * i)))
    dl = lt.data.DataLoader(Sq(), 4, False, lt.Device("cpu"), 2)
    assert len(Sq()) == 10
    ys = [v for b in dl for v in _unwrap(b[1]).tolist()]
    assert ys == [float(i * i) for i in range(10)]


# ------------------------------------------------------------------ JIT
def test_jit_tree_derivative_serialisation_and_autograd(tmp_path):
    J = lt.jit
    x, y = J.JITVar.input("x"), J.JITVar.input("y")
    f = J.JITFunction("f", J.gelu(x * y) + J.sigmoid(x) / 2.0 - J.abs(y), [x, y])
    a = lt.Tensor(torch.randn(7, requires_grad=True))
    b = lt.Tensor(torch.randn(7, requires_grad=True))
    out = f(a, b)
    ta, tb = _unwrap(a).detach().requires_grad_(True), _unwrap(b).detach().requires_grad_(True)
    ref = torch.nn.functional.gelu(ta * tb, approximate="tanh") + torch.sigmoid(ta) / 2 - tb.abs()
    assert torch.allclose(_unwrap(out), ref, atol=1e-5)
    lt.Ops.sum(out).backward()
    ref.sum().backward()
    assert torch.allclose(_unwrap(a).grad, ta.grad, atol=1e-4) and torch.allclose(_unwrap(b).grad, tb.grad, atol=1e-4)
    d = J.Tracer.derivative(x * x * x, "x")
    df = J.JITFunction("d", d, [x])
    assert _unwrap(df(lt.Tensor(torch.tensor([2.0])))).item() == pytest.approx(12.0)
    path = str(tmp_path / "f.txt")
    f.save(path)
    lines = open(path).read().split("\n")
    assert lines[0] == "f" and lines[1] == "2" and lines[2:4] == ["x", "y"] and lines[4].startswith("3 _ 0 ")
    g = J.JITFunction.load(path)
    assert torch.allclose(_unwrap(g(a, b)), _unwrap(out))
    old = J.Tracer.deserialize_var("(6,,0,(4,,0,(0,x,0,N,N),(0,y,0,N,N)),N)")      # parenthesised form of saved files
    assert old.op == J.OpType.RELU and old.left.op == J.OpType.MUL and old.left.left.name == "x"
    r = J.fused_bias_gelu(lt.Tensor(torch.ones(2, 3)), lt.Tensor(torch.tensor([0.0, 1.0, 2.0])))
    assert torch.allclose(_unwrap(r), torch.nn.functional.gelu(torch.ones(2, 3) + torch.tensor([0., 1., 2.]), approximate="tanh"), atol=1e-5)
    assert _unwrap(J.fused_residual_add(lt.Tensor(torch.ones(3)), lt.Tensor(torch.ones(3)))).tolist() == [2.0] * 3


# ------------------------------------------------------------------ serving
class _NextTok(lt.nn.Module):
    """Mock LM: next token = (last token + 1) % V (the reference tests use the same mock)."""

    def __init__(self, V=16):
        super().__init__()
        self.V = V

    def forward(self, x):
        t = _unwrap(x).long()
        return lt.Tensor(torch.nn.functional.one_hot((t + 1) % self.V, self.V).float())


def test_continuous_batching_admission_chunked_prefill_and_recycling():
    S = lt.nn.ServingScheduler(num_blocks=8, block_size=4, max_num_seqs=4, max_num_batched_tokens=6)
    reqs = [lt.nn.Request(i, [3, 4, 5, 6, 7], max_new_tokens=3) for i in range(5)]
    for r in reqs:
        S.add_request(r)
    model, done, steps = _NextTok(), [], 0
    while len(done) < 5 and steps < 100:
        done += S.step(model)
        steps += 1
        assert S.free_blocks + sum(len(r.block_ids) for r in S.running_queue) == 8
    assert len(done) == 5 and all(r.is_finished for r in reqs)
    assert all(r.generated_tokens == [8, 9, 10] for r in reqs)
    assert S.free_blocks == 8
    # each request needs ceil((5+3)/4) = 2 blocks, so at most 4 run at once and the fifth waits
    S2 = lt.nn.ServingScheduler(4, 4, 8, 64)
    for i in range(3):
        S2.add_request(lt.nn.Request(i, [1, 2, 3, 4, 5], 3))
    S2.step(model)
    assert len(S2.running_queue) == 2 and len(S2.pending_queue) == 1
    assert S2.get_block_table_tensor().shape == [2, 2] and S2.get_context_lens_tensor().shape == [2]
    eos = lt.nn.ServingScheduler(8, 4, 2, 64)
    eos.add_request(lt.nn.Request(0, [15, 0], max_new_tokens=10))   # 0 -> 1 -> 2 (EOS)
    out = []
    for _ in range(10):
        out += eos.step(model)
    assert out and out[0].generated_tokens == [1, 2]


def test_prefix_cache_speculative_medusa_guided():
    pc = lt.nn.PrefixCache.get()
    pc.clear()
    kv = [lt.Tensor(torch.ones(2, 2))]
    pc.put([1, 2, 3, 4], kv, blocks=[7, 9])
    assert pc.get_cache([1, 2, 3, 4]) == kv and pc.get_cache([1, 2]) == []
    assert pc.longest_prefix([1, 2, 3, 4, 5, 6], granularity=2) == (4, [7, 9])
    assert pc.longest_prefix([9, 9], 1) == (0, [])
    m = _NextTok()
    spec = lt.nn.SpeculativeEngine(m, m)
    assert spec.generate([1, 2], 6, lookahead=3) == [1, 2, 3, 4, 5, 6, 7, 8]

    class Bad(_NextTok):
        def forward(self, x):
            return lt.Tensor(torch.nn.functional.one_hot((_unwrap(x).long() + 2) % self.V, self.V).float())
    assert lt.nn.SpeculativeEngine(Bad(), m).generate([1], 4, 2) == [1, 2, 3, 4, 5]      # all drafts rejected
    heads = [lt.nn.MedusaHead(16, 16) for _ in range(2)]
    assert lt.nn.MedusaEngine(m, heads).generate([5], 4, 2)[:5] == [5, 6, 7, 8, 9]
    gd = lt.nn.GuidedDecoder(["1", "a", "23", "b4", "hello", "he"])
    lg = lt.Tensor(torch.zeros(6))
    gd.apply_mask(lg, "4", "digits")
    assert _unwrap(lg).tolist() == [0, -1e9, 0, -1e9, -1e9, -1e9]
    lg = lt.Tensor(torch.zeros(6))
    gd.apply_mask(lg, "", "prefix:hello")
    assert [v == 0 for v in _unwrap(lg).tolist()] == [False, False, False, False, True, True]
    lg = lt.Tensor(torch.zeros(6))
    gd.apply_mask(lg, "x", "regex:^x[a-z]+$")
    assert [v == 0 for v in _unwrap(lg).tolist()] == [False, True, False, False, True, True]


# ------------------------------------------------------------------ allocator, LRU, thread pool
def test_caching_allocator_and_lru_manager():
    import ctypes
    from litetorch_b200._native import host_lib
    L = host_lib()
    L.lt_pool_create.restype = ctypes.c_void_p
    L.lt_pool_alloc.restype = ctypes.c_void_p
    L.lt_pool_create.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_uint64] * 3
    L.lt_pool_alloc.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
    L.lt_pool_free.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    L.lt_pool_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64)]
    L.lt_pool_empty_cache.argtypes = [ctypes.c_void_p]
    L.lt_pool_destroy.argtypes = [ctypes.c_void_p]
    pool = L.lt_pool_create(None, None, None, 1 << 20, 0, 512)
    a = L.lt_pool_alloc(pool, 4000)
    L.lt_pool_free(pool, a)
    b = L.lt_pool_alloc(pool, 3000)        # reuses the 4096-byte block (<= 2x the rounded request)
    assert a == b
    L.lt_pool_free(pool, b)
    c = L.lt_pool_alloc(pool, 100)         # 4096 > 2 * 512: no reuse
    assert c != a
    st = (ctypes.c_uint64 * 6)()
    L.lt_pool_stats(pool, st)
    assert st[4] == 1 and st[5] == 2 and st[0] == 4096
    L.lt_pool_free(pool, c)
    L.lt_pool_empty_cache(pool)
    L.lt_pool_stats(pool, st)
    assert st[0] == 0
    L.lt_pool_destroy(pool)
    # LRU: limit 100, three storages of 40 -> registering the third evicts the least recently used idle one
    L.lt_lru_create.restype = ctypes.c_void_p
    L.lt_lru_create.argtypes = [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    L.lt_lru_register.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64), ctypes.c_int]
    L.lt_lru_touch.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
    L.lt_lru_pin.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int]
    L.lt_lru_used.restype = ctypes.c_uint64
    L.lt_lru_used.argtypes = [ctypes.c_void_p]
    lru = L.lt_lru_create(100, None, None)
    ev = (ctypes.c_uint64 * 4)()
    assert L.lt_lru_register(lru, 1, 40, ev, 4) == 0 and L.lt_lru_register(lru, 2, 40, ev, 4) == 0
    L.lt_lru_touch(lru, 1)                 # 2 is now the oldest
    assert L.lt_lru_register(lru, 3, 40, ev, 4) == 1 and ev[0] == 2
    L.lt_lru_pin(lru, 1, 1)                # pinned storages are skipped
    assert L.lt_lru_register(lru, 4, 40, ev, 4) == 1 and ev[0] == 3 and L.lt_lru_used(lru) == 80


def test_tcp_store_barrier_heartbeat_and_dead_rank_detection():
    from litetorch_b200.parallel.process_group import RankFailure, TCPStore, Watchdog
    server = TCPStore("127.0.0.1", 0, is_server=True)
    peer = TCPStore("127.0.0.1", server.port, is_server=False)
    server.set("id", b"\x01\x02\x03")
    assert peer.get("id") == b"\x01\x02\x03"
    with pytest.raises(TimeoutError):
        peer.get("never", timeout_s=0.2)
    assert peer.add("ctr", 5) == 5 and server.add("ctr", 2) == 7
    res = []
    t = threading.Thread(target=lambda: res.append(peer.barrier("b", 2, 5.0)))
    t.start()
    server.barrier("b", 2, 5.0)
    t.join()
    with pytest.raises(TimeoutError):
        server.barrier("lonely", 2, 0.2)                 # the other rank never joins
    w0 = Watchdog(server, 0, interval_s=0.05, ttl_s=0.4)
    w1 = Watchdog(peer, 1, interval_s=0.05, ttl_s=0.4)
    time.sleep(0.2)
    w0.check()
    w1.stop()                                            # rank 1 stops answering
    time.sleep(0.7)
    with pytest.raises(RankFailure, match=r"\[1\]"):
        w0.check()
    w0.stop()
    peer.close()
    server.close()


def test_file_store(tmp_path):
    from litetorch_b200.parallel.process_group import FileStore
    fs = FileStore(str(tmp_path / "rdv"))
    fs.set("nccl_id", b"x" * 128)
    assert fs.get("nccl_id") == b"x" * 128
    with pytest.raises(TimeoutError):
        fs.get("missing", timeout_s=0.1)


def test_store_delayed_rendezvous_lost_server_and_unreachable_host():
    """Host-side fault injection on the rendezvous store: a client that starts before the server keeps retrying and gets
    through; a client of a server that has gone away gets an error instead of hanging; nobody listening is a timeout."""
    import socket
    import threading
    import time
    from litetorch_b200.parallel.process_group import TCPStore
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()                                              # a free port nobody listens on yet
    got = {}

    def late_client():
        c = TCPStore("127.0.0.1", port, is_server=False, timeout_s=10.0)     # the server is not up yet
        got["v"] = c.get("ready", timeout_s=10.0)
        c.close()
    t = threading.Thread(target=late_client)
    t.start()
    time.sleep(1.0)                                        # the delayed rendezvous
    server = TCPStore("127.0.0.1", port, is_server=True)
    server.set("ready", b"yes")
    t.join(timeout=20)
    assert not t.is_alive() and got.get("v") == b"yes"
    # the server goes away under a connected client
    client = TCPStore("127.0.0.1", port, is_server=False, timeout_s=5.0)
    client.set("k", b"1")
    server.close()
    t0 = time.time()
    with pytest.raises((RuntimeError, TimeoutError)):
        client.get("never", timeout_s=3.0)
    assert time.time() - t0 < 10
    client.close()
    # nobody listening: connecting gives up after its timeout
    t0 = time.time()
    with pytest.raises(RuntimeError):
        TCPStore("127.0.0.1", port, is_server=False, timeout_s=1.0)
    assert 0.5 < time.time() - t0 < 5


def test_store_edge_cases_of_rendezvous_and_failure_detection():
    """Four host-side failure paths of the native store: a rank that dies before its first heartbeat is reported once
    the grace period is over; a barrier that timed out leaves the counter usable for the next barrier; a client that
    disconnects does not leave a stale descriptor behind for the server's stop path; a client whose request timed out
    drops its connection instead of reading the tail of the old answer."""
    import socket
    import threading
    import time
    from litetorch_b200.parallel.process_group import RankFailure, TCPStore, Watchdog
    server = TCPStore("127.0.0.1", 0, is_server=True)
    # ---- 1. rank 1 of a world of 2 never starts: invisible to dead_ranks, reported through silent_ranks after the grace period
    w0 = Watchdog(server, 0, interval_s=0.05, ttl_s=0.5, world_size=2, grace_s=0.3)
    time.sleep(0.15)
    w0.check()                                     # inside the grace period: nothing to report yet
    assert server.dead_ranks(0.5) == []
    time.sleep(0.3)
    with pytest.raises(RankFailure):
        w0.check()
    assert server.silent_ranks(2, 0.5) == [1]
    w0.stop()
    # ---- 2. a barrier nobody else joins times out; the next barrier on the same key, with both ranks, completes
    peer = TCPStore("127.0.0.1", server.port, is_server=False)
    with pytest.raises(TimeoutError):
        server.barrier("b", 2, timeout_s=0.2)
    done = []
    t = threading.Thread(target=lambda: (peer.barrier("b", 2, timeout_s=5.0), done.append(1)))
    t.start()
    server.barrier("b", 2, timeout_s=5.0)
    t.join(timeout=5)
    assert done == [1]
    # ---- 3. a client disconnects; descriptors opened afterwards must survive the server's stop
    peer.close()
    time.sleep(0.1)
    a, b = socket.socketpair()                     # likely reuses the descriptor number the server just closed
    # ---- 4. a request that times out closes the client's connection
    mute = socket.socket()
    mute.bind(("127.0.0.1", 0))
    mute.listen(1)                                 # accepts the connection but never answers
    c = TCPStore("127.0.0.1", mute.getsockname()[1], is_server=False, timeout_s=2.0)
    c._lib.lt_store_set_timeout(c._c, 200)
    assert c.alive()
    with pytest.raises(Exception):
        c.set("k", b"v")                           # no answer within 200 ms
    assert not c.alive()                           # the half-finished exchange is gone with the connection
    with pytest.raises(Exception):
        c.set("k", b"v")                           # and later calls fail at once instead of parsing stale bytes
    server.close()
    a.send(b"x")
    assert b.recv(1) == b"x"                       # the unrelated socket pair was not shut down by the stop path
    a.close(); b.close(); mute.close()


def test_residency_manager_evicts_to_host_and_swaps_back_in_under_a_2mb_limit():
    """Sixteen 512 KB tensors under a 2 MB limit (the reference's stress test uses the same limit,
    tests/stress_test.cpp:36-70): at most four are resident, the others wait on the host and come back intact in LRU
    order; a tensor in use is never the victim; AdamW with its moments under a limit takes the same steps as without."""
    import litetorch_b200 as lt
    from litetorch_b200.core import Tensor, _unwrap
    mm = lt.memory.ResidencyManager(2 << 20, device="cpu")
    hs = [mm.register(torch.full((128 * 1024,), float(i))) for i in range(16)]
    assert mm.resident_bytes <= 2 << 20 and sum(h.resident for h in hs) == 4 and mm.evictions == 12
    assert [h.resident for h in hs[-4:]] == [True] * 4
    for i, h in enumerate(hs):                      # every tensor comes back with its contents
        assert float(mm.fetch(h)[777]) == float(i)
        assert mm.resident_bytes <= 2 << 20
    assert mm.swap_ins == 12 + 4 - 4 or mm.swap_ins >= 12
    with mm.use(hs[0]) as t0:                       # pinned: stays while four others are brought in
        for h in hs[1:6]:
            mm.fetch(h)
        assert hs[0].resident and t0 is hs[0].tensor
    mm.release(hs[3])
    # AdamW: moments of 6 x 256 KB parameters under a 1 MB limit follow the unlimited optimizer exactly
    def run(limit):
        g = torch.Generator().manual_seed(0)
        ps = [Tensor(torch.randn(64 * 1024, generator=g).requires_grad_(True)) for _ in range(6)]
        opt = lt.optim.AdamW(ps, lr=1e-2, weight_decay=0.1, state_limit_bytes=limit)
        for step in range(3):
            for k, p in enumerate(ps):
                _unwrap(p).grad = torch.full((64 * 1024,), 0.1 * (k + 1) * (step + 1))
            opt.step()
        return [_unwrap(p).detach().clone() for p in ps], opt
    free, _ = run(0)
    lim, opt = run(1 << 20)
    assert all(torch.equal(a, b) for a, b in zip(free, lim))
    assert opt._mm.evictions > 0 and opt._mm.resident_bytes <= 1 << 20

"""Every name of the reference's Python binding (src/bindings/python_bindings.cpp:91-966) exists in this package."""
import litetorch_b200 as lt

SURFACE = {
    "": "DeviceType Device is_gpu_available auto_device get_backend_name DataType Tensor checkpoint save load save_parameters "
        "load_parameters save_optimizer_state load_optimizer_state empty_cache set_max_cpu_cache_size get_cached_cpu_bytes "
        "get_cached_gpu_bytes get_gpu_memory_used",
    "Tensor": "create from_vector zeros shape strides dtype device requires_grad grad numel item to_vector backward zero_grad to "
              "view reshape transpose contiguous is_contiguous clone cast copy_ add_ register_hook",
    "cuda": "is_available set_tf32_enabled is_tf32_enabled memory_allocated",
    "Ops": "add sub mul div matmul bmm sum mean max pow sqrt exp log abs neg clamp sin cos relu leaky_relu sigmoid tanh softmax "
           "gelu layer_norm fused_add_layernorm batch_norm2d conv2d conv3d max_pool2d max_pool3d adaptive_avg_pool2d cat squeeze "
           "unsqueeze cast fake_quantize mse_loss cross_entropy_loss l1_loss bce_loss fused_linear_cross_entropy clip_grad_norm_ "
           "rope flash_attention paged_attention scaled_matmul w8a8_matmul moe_gate flash_decoding ring_attention checkpoint",
    "nn": "Module Linear QLoRALinear MoELinear ColumnParallelLinear RowParallelLinear Conv2d Conv3d BatchNorm2d MaxPool2d "
          "MaxPool3d AdaptiveAvgPool2d Dropout ReLU LeakyReLU Sigmoid Tanh GELU Softmax Flatten Embedding LayerNorm "
          "MultiHeadAttention TransformerDecoderLayer Sequential MSELoss CrossEntropyLoss BCELoss L1Loss GuidedDecoder Request "
          "ServingScheduler PrefixCache SpeculativeEngine MedusaHead MedusaEngine",
    "optim": "Optimizer SGD Adam AdamW AdamW8bit AdamWFP8 RMSprop ZeRO3Optimizer StepLR CosineAnnealingLR GradScaler",
    "amp": "GradScaler AutocastGuard",
    "quantization": "quantize_linear Calibrator QATLinear",
    "distributed": "ProcessGroup DeviceMesh PlacementType Placement DTensor FullyShardedDataParallel OverlappedAllReducer "
                   "overlapped_all_reduce overlapped_reduce_scatter sync_overlapped_all_reduce PipelineParallelModule FSDP "
                   "init_process_group manual_seed",
    "distributed.PipelineParallelModule": "forward forward_microbatches schedule_1f1b train_step_1f1b run_1f1b_with_backward "
                                          "parameters to",
    "distributed.FullyShardedDataParallel": "gather_parameters shard_parameters get_module",
    "jit": "OpType JITVar relu gelu sigmoid tanh sqrt exp log abs fused_bias_relu fused_bias_gelu fused_residual_add "
           "fused_residual_gelu JITFunction Tracer",
    "jit.Tracer": "trace derivative serialize_var deserialize_var",
    "jit.JITFunction": "__call__ forward save load",
    "data": "Dataset TensorDataset DataLoader",
    "data.DataLoader": "reset next save_state load_state",
}


def test_reference_python_surface_is_present():
    missing = []
    for where, names in SURFACE.items():
        obj = lt
        for part in filter(None, where.split(".")):
            obj = getattr(obj, part)
        missing += [(where + "." + n).lstrip(".") for n in names.split() if not hasattr(obj, n)]
    pg = lt.distributed.ProcessGroup.get()
    missing += ["ProcessGroup." + n for n in ("init shutdown all_reduce broadcast all_gather reduce_scatter send_tensor recv_tensor "
                                              "sync_comm get_rank get_world_size is_initialized").split() if not hasattr(pg, n)]
    assert not missing, missing
    assert hasattr(lt.DataType, "FP4") and hasattr(lt.distributed.FSDP, "fully_shard")


def test_a_script_written_for_the_reference_runs_unchanged(tmp_path):
    """`python -m litetorch_b200.compat script.py` binds the name `litetorch`: the calls the reference's own Python test makes
    (tests/test_litetorch.py: from_vector / add / sum / backward, Linear + AdamW + mse_loss, the function form of checkpoint)."""
    import json
    import os
    import subprocess
    import sys
    script = tmp_path / "user_script.py"
    script.write_text('''
import json
import litetorch as lt
from litetorch import nn
dev = lt.Device("cpu")
x = lt.Tensor.from_vector([1.0, 2.0, 3.0, 4.0], [2, 2], dev, True)
y = lt.Tensor.from_vector([2.0, 0.5, 1.0, 2.0], [2, 2], dev, True)
z = lt.Ops.add(x, y)
loss = lt.Ops.sum(z)
loss.backward()
lin = nn.Linear(2, 1, True)
opt = lt.optim.AdamW(lin.parameters(), lr=0.01)
out = lin.forward(lt.Tensor.from_vector([1.0, 2.0], [1, 2], dev, False))
mse = lt.Ops.mse_loss(out, lt.Tensor.from_vector([5.0], [1, 1], dev, False))
before = [p.to_vector() for p in lin.parameters()]
opt.zero_grad(); mse.backward(); opt.step()
after = [p.to_vector() for p in lin.parameters()]
xc = lt.Tensor.from_vector([1.0, 2.0, 3.0, 4.0], [4], dev, True)
cp = lt.checkpoint(lambda t: lt.Ops.add(lt.Ops.mul(t, t), t), xc)
lt.Ops.sum(cp).backward()
print("RESULT " + json.dumps({"z": z.to_vector(), "sum": loss.item(), "gx": x.grad.to_vector(), "moved": before != after,
                              "gcp": xc.grad.to_vector(), "mse": mse.item()}))
''')
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "litetorch_b200.compat", str(script)], capture_output=True, text=True, timeout=300,
                       cwd=root)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["z"] == [3.0, 2.5, 4.0, 6.0] and res["sum"] == 15.5 and res["gx"] == [1.0, 1.0, 1.0, 1.0]
    assert res["moved"] and res["gcp"] == [3.0, 5.0, 7.0, 9.0] and res["mse"] > 0


def test_the_example_applications_call_patterns_work():
    """The call shapes of the reference's example applications (train_cat_dog_cnn.py / train_cat_dog.py): positional Conv2d /
    MaxPool2d / Linear arguments, JIT functions called with a list, reshape with a list, `.forward`, parameter lists that are
    concatenated, `.to(device)`, dropout train / eval, cross-entropy on float class ids, save / load of a module."""
    import os
    import tempfile
    import torch
    import litetorch_b200 as lt

    class Net(lt.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1, self.p1 = lt.nn.Conv2d(3, 8, 3, 1, 1, True), lt.nn.MaxPool2d(2, 2, 0)
            self.c2, self.p2 = lt.nn.Conv2d(8, 16, 3, 1, 1, True), lt.nn.MaxPool2d(2, 2, 0)
            self.drop = lt.nn.Dropout(0.3)
            self.norm = lt.nn.LayerNorm([16 * 4 * 4])
            self.fc1, self.fc2 = lt.nn.Linear(16 * 4 * 4, 32, True), lt.nn.Linear(32, 2, True)
            v1, v2 = lt.jit.JITVar(lt.jit.OpType.INPUT, "a"), lt.jit.JITVar(lt.jit.OpType.INPUT, "b")
            self.r1 = lt.jit.JITFunction("relu_a", lt.jit.relu(v1), [v1])
            self.r2 = lt.jit.JITFunction("relu_b", lt.jit.relu(v2), [v2])

        def forward(self, x):
            b = x.shape[0]
            h = self.p1.forward(self.r1([self.c1.forward(x)]))
            h = self.p2.forward(self.r2([self.c2.forward(h)]))
            h = self.drop.forward(h).reshape([b, 16 * 4 * 4])
            return self.fc2.forward(lt.Ops.gelu(self.fc1.forward(self.norm.forward(h))))

        def parameters(self):
            return self.c1.parameters() + self.c2.parameters() + self.norm.parameters() + self.fc1.parameters() + self.fc2.parameters()

        def to(self, device):
            for m in (self.c1, self.c2, self.norm, self.fc1, self.fc2):
                m.to(device)

    lt.manual_seed(0)
    dev = lt.auto_device() if not lt.is_gpu_available() else lt.Device("cpu")
    net = Net()
    net.to(dev)
    net.drop.eval()
    g = torch.Generator().manual_seed(0)
    imgs = torch.randn(8, 3, 16, 16, generator=g)
    labels = (imgs.mean((1, 2, 3)) > 0).float()
    x = lt.Tensor.from_vector(imgs.flatten().tolist(), [8, 3, 16, 16], dev, False)
    y = lt.Tensor.from_vector(labels.tolist(), [8], dev, False)
    opt = lt.optim.AdamW(net.parameters(), lr=3e-3)
    losses = []
    for _ in range(30):
        opt.zero_grad()
        loss = lt.Ops.cross_entropy_loss(net.forward(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.5 * losses[0], losses
    probs = lt.Ops.softmax(net.forward(x), -1).to_vector()
    assert len(probs) == 16 and abs(sum(probs[:2]) - 1.0) < 1e-5
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "net.ltw")
        lt.save(net, path)
        before = [p.to_vector() for p in net.parameters()]
        for p in net.parameters():
            p.add_(lt.Tensor.from_vector([1.0] * p.numel(), p.shape, dev, False))
        lt.load(net, path)
        assert [p.to_vector() for p in net.parameters()] == before
    lt.empty_cache()
    assert isinstance(lt.get_backend_name(), str) and lt.get_gpu_memory_used() >= 0 and lt.cuda.memory_allocated() >= 0


def test_the_vit_example_call_patterns_work():
    """Call shapes of the reference's ViT example (train_cat_dog.py): MultiHeadAttention(embed, heads).forward on [B, N, E],
    LayerNorm([E]), a learned position tensor added by broadcasting, transpose(1, 2) followed by a Linear over the patch
    axis, contiguous().view([B, E]), parameter lists that include a bare Tensor."""
    import torch
    import litetorch_b200 as lt
    B, N, P, E, H = 4, 16, 12, 32, 4
    dev = lt.Device("cpu")
    lt.manual_seed(1)

    class Block(lt.nn.Module):
        def __init__(self):
            super().__init__()
            self.attn, self.ln1, self.ln2 = lt.nn.MultiHeadAttention(E, H), lt.nn.LayerNorm([E]), lt.nn.LayerNorm([E])
            self.fc1, self.fc2 = lt.nn.Linear(E, 2 * E, True), lt.nn.Linear(2 * E, E, True)

        def forward(self, x):
            x = lt.Ops.add(x, self.attn.forward(self.ln1.forward(x)))
            return lt.Ops.add(x, self.fc2.forward(lt.Ops.gelu(self.fc1.forward(self.ln2.forward(x)))))

        def parameters(self):
            return self.attn.parameters() + self.ln1.parameters() + self.fc1.parameters() + self.fc2.parameters() + self.ln2.parameters()

    proj, blk, ln_f = lt.nn.Linear(P, E, True), Block(), lt.nn.LayerNorm([E])
    pool, head = lt.nn.Linear(N, 1, False), lt.nn.Linear(E, 2, True)
    pos = lt.Tensor.from_vector((torch.randn(N * E) * 0.02).tolist(), [1, N, E], dev, True)

    def forward(x):
        h = ln_f.forward(blk.forward(lt.Ops.add(proj.forward(x), pos)))
        return head.forward(pool.forward(h.transpose(1, 2)).contiguous().view([B, E]))

    params = proj.parameters() + [pos] + blk.parameters() + ln_f.parameters() + pool.parameters() + head.parameters()
    opt = lt.optim.AdamW(params, lr=3e-3)
    g = torch.Generator().manual_seed(2)
    xs = torch.randn(B, N, P, generator=g)
    x = lt.Tensor.from_vector(xs.flatten().tolist(), [B, N, P], dev, False)
    y = lt.Tensor.from_vector([0.0, 1.0, 1.0, 0.0], [B], dev, False)
    losses = []
    for _ in range(40):
        opt.zero_grad()
        loss = lt.Ops.cross_entropy_loss(forward(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert pos.grad is not None and losses[-1] < 0.3 * losses[0], losses


def test_keyword_names_and_fields_of_the_reference_bindings():
    """Keyword names (py::arg) and read-write fields (def_readwrite) of src/bindings/python_bindings.cpp that differ from the
    obvious Python spelling: each must be accepted / present here too."""
    import inspect
    import torch
    import litetorch_b200 as lt
    from litetorch_b200 import data as DT, distributed as D, jit as J, nn, optim, quantization as Q

    def accepts(fn, *names):
        ps = inspect.signature(fn).parameters
        return all(n in ps for n in names)

    assert accepts(lt.Tensor.cast, "target_dtype") and accepts(lt.Ops.cast, "a", "target_dtype")
    for f in ("layer_norm", "fused_add_layernorm", "batch_norm2d", "conv2d", "conv3d", "max_pool2d", "max_pool3d", "adaptive_avg_pool2d",
              "fake_quantize"):
        assert accepts(getattr(lt.Ops, f), "input"), f
    assert accepts(lt.Ops.checkpoint, "module", "input")
    assert accepts(lt.save_optimizer_state, "optimizer", "filepath") and accepts(lt.load_optimizer_state, "optimizer", "filepath")
    assert accepts(D.ProcessGroup.recv_tensor, "tensor", "src") and accepts(D.overlapped_all_reduce, "tensor")
    assert accepts(D.DeviceMesh.get_rank, "coords") and accepts(D.DTensor.redistribute, "new_mesh", "new_placements")
    assert accepts(D.PipelineParallelModule.forward, "input") and accepts(DT.Dataset.__getitem__, "index")
    assert accepts(J.JITVar.__init__, "op", "name", "val") and accepts(J.Tracer.deserialize_var, "str")
    assert accepts(Q.QATLinear.__init__, "linear", "w_scale", "w_zp", "a_scale", "a_zp", "b")

    lin = nn.Linear(4, 4, True)
    opt = optim.AdamW(lin.parameters(), lr=0.5)
    opt.set_lr(new_lr=0.25)
    assert opt.get_lr() == 0.25 and opt.lr == 0.25
    for cls in (optim.SGD, optim.Adam, optim.AdamW8bit, optim.AdamWFP8, optim.RMSprop):
        o = cls(lin.parameters())
        o.set_lr(0.125)
        assert o.get_lr() == 0.125
    sch = optim.StepLR(opt, step_size=2, gamma=0.5)
    for _ in range(2):
        sch.step()
    assert sch.last_epoch == 2 and opt.lr == 0.125
    cos = optim.CosineAnnealingLR(opt, T_max=4, eta_min=0.0)
    cos.step()
    assert cos.last_epoch == 1
    assert Q.QATLinear(lin, b=4).bits == 4 and J.JITVar(val=2.0).val == 2.0 and J.JITVar(op=J.OpType.INPUT, name="q").name == "q"
    fields = [(nn.QLoRALinear(4, 4), ["weight", "bias", "lora_A", "lora_B", "scaling"]),
              (nn.BatchNorm2d(2), ["num_features", "eps", "momentum", "running_mean", "running_var"]),
              (nn.MaxPool2d(2, 2, 0), ["kernel_size", "stride", "padding"]), (nn.MaxPool3d(2), ["kernel_size", "stride", "padding"]),
              (nn.AdaptiveAvgPool2d(1, 1), ["output_height", "output_width"]), (nn.Embedding(5, 3), ["num_embeddings", "embedding_dim", "weight"]),
              (nn.LayerNorm([4]), ["weight", "bias", "eps", "normalized_shape"]), (nn.MultiHeadAttention(8, 2), ["embed_dim", "num_heads", "head_dim"])]
    for obj, names in fields:
        assert all(hasattr(obj, n) for n in names), (type(obj).__name__, names)
    mesh = D.DeviceMesh([2, 2], "tp,dp", rank=0, create_groups=False)
    assert mesh.mesh_shape == [2, 2] and mesh.mesh_dim_names == "tp,dp" and mesh.mesh_topology == [0, 1, 2, 3]
    assert mesh.get_rank() == 0 and mesh.get_rank(coords=[1, 0]) == 2
    pl = D.Placement()
    pl.type, pl.dim = D.PlacementType.SHARD, 0
    dt = D.DTensor(lt.Tensor(torch.ones(2, 2)), mesh, [pl])                  # one placement on a 2-D mesh: the rest replicate
    assert dt.device_mesh is mesh and len(dt.placements) == 2
    same = dt.redistribute(mesh, dt.placements)
    assert same.placements == dt.placements


def test_tracer_follows_the_reference_form():
    """`Tracer.trace([tensors], fn(list) -> Tensor, name)` records the lt.Ops calls between the example tensors
    (src/ops/jit.cpp:496-525); the symbolic form with input names keeps working."""
    import torch
    import litetorch_b200 as lt
    from litetorch_b200.core import _unwrap
    dev = lt.Device("cpu")
    a = lt.Tensor.from_vector([1.0, -2.0, 3.0], [3], dev, False)
    b = lt.Tensor.from_vector([0.5, 1.5, -2.0], [3], dev, False)
    fn = lt.jit.Tracer.trace([a, b], lambda args: lt.Ops.gelu(lt.Ops.add(lt.Ops.mul(args[0], args[1]), args[0])), "fused")
    got = _unwrap(fn([a, b]))
    ref = torch.nn.functional.gelu(_unwrap(a) * _unwrap(b) + _unwrap(a), approximate="tanh")
    assert torch.allclose(got, ref, atol=1e-5) and fn.input_names == ["x0", "x1"]
    x2 = lt.Tensor.from_vector([2.0, 0.0, -1.0], [3], dev, True)
    out = fn([x2, b])
    lt.Ops.sum(out).backward()
    assert x2.grad is not None
    sym = lt.jit.Tracer.trace(["x", "w"], lambda x, w: lt.jit.relu(x * 2.0 + w), "sym")
    assert _unwrap(sym([a, b])).tolist() == [2.5, 0.0, 4.0]
    import pytest
    with pytest.raises(ValueError):
        lt.jit.Tracer.trace([a], lambda args: lt.Ops.softmax(args[0], -1), "unsupported")


def test_enum_values_are_exported_into_their_modules():
    import litetorch_b200 as lt
    assert lt.distributed.SHARD is lt.distributed.PlacementType.SHARD and lt.distributed.PARTIAL is lt.distributed.PlacementType.PARTIAL
    assert lt.jit.INPUT is lt.jit.OpType.INPUT and lt.jit.GELU is lt.jit.OpType.GELU and callable(lt.jit.gelu)
    assert lt.CPU is lt.DeviceType.CPU and lt.FP32 is lt.DataType.FP32


def test_scheduler_step_without_a_model_plans_only():
    """The reference's serving guide calls `scheduler.step()` and then reads the block tables: admission and planning
    happen, no position moves, and a later `step(model)` serves the request as usual."""
    import torch
    s = lt.nn.ServingScheduler(num_blocks=8, block_size=4, max_num_seqs=2, max_num_batched_tokens=16)
    r = lt.nn.Request(id=1, prompt=[1, 2, 3, 4, 5], max_new_tokens=2)
    s.add_request(r)
    first, second = s.step(), s.step()
    assert [q.id for q in first] == [1] == [q.id for q in second] and len(r.block_ids) == 2 and s.free_blocks == 6
    assert s.get_block_table_tensor().shape == [1, 2] and s.get_context_lens_tensor().to_vector() == [0.0]

    class Next(lt.nn.Module):
        def forward(self, x):
            return lt.Tensor(torch.nn.functional.one_hot((x.torch().long() + 1) % 16, 16).float())
    while not r.is_finished:
        s.step(Next())
    assert r.generated_tokens == [6, 7] and s.free_blocks == 8

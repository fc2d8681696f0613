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

"""Expected values that the reference's own C++ tests assert, replayed through this package's Python API on the CPU
(tests/stage4_test.cpp: asymmetric calibration + fake quantisation, JIT forward / saved / derivative functions;
tests/audit_bugs_test.cpp: conv3d on a transposed view, gradient accumulation when a tensor is used twice)."""
import litetorch_b200 as lt

CPU = lt.Device("cpu")


def _t(v, shape, grad=False):
    return lt.Tensor.from_vector([float(x) for x in v], shape, CPU, grad)


def test_asymmetric_calibration_and_fake_quantize():
    t = _t([-10.0, -5.0, 0.0, 2.0], [4])
    cal = lt.quantization.Calibrator()
    cal.collect("test_layer", t)
    scale, zp = cal.get_asymmetric_params("test_layer", 8)
    assert scale > 0.0 and -127.0 <= zp <= 127.0
    q = lt.Ops.fake_quantize(t, scale, zp, 8).to_vector()
    assert abs(q[0] + 10.0) < 0.1 and abs(q[3] - 2.0) < 0.1


def test_jit_forward_saved_and_derivative_functions(tmp_path):
    J = lt.jit
    x, y = J.JITVar(J.OpType.INPUT, "x"), J.JITVar(J.OpType.INPUT, "y")
    expr = J.relu(x * y)
    fwd = J.JITFunction("fwd", expr, [x, y])
    bwd = J.JITFunction("bwd", J.Tracer.derivative(expr, x), [x, y])
    x1, y1 = _t([-2, 3, 4, -5], [4]), _t([2, 2, -2, 2], [4])
    assert fwd([x1, y1]).to_vector() == [0.0, 6.0, 0.0, 0.0]
    path = str(tmp_path / "jit_func_test.txt")
    fwd.save(path)
    assert J.JITFunction.load(path)([x1, y1]).to_vector() == [0.0, 6.0, 0.0, 0.0]
    assert bwd([x1, y1]).to_vector() == [0.0, 2.0, 0.0, 0.0]
    # another length through the same functions (the reference guards its compiled kernels by shape)
    x2, y2 = _t([-1, 2, 3, 4, 5, -6], [6]), _t([3, 3, 3, 3, -3, 3], [6])
    assert fwd([x2, y2]).to_vector() == [0.0, 6.0, 9.0, 12.0, 0.0, 0.0]
    assert bwd([x2, y2]).to_vector() == [0.0, 3.0, 3.0, 3.0, 0.0, 0.0]


def test_conv3d_reads_a_transposed_view_correctly():
    inp = _t([1, 2, 3, 4, 5, 6, 7, 8], [1, 1, 2, 2, 2]).transpose(3, 4)
    assert not inp.is_contiguous()
    out = lt.Ops.conv3d(inp, _t([1.0], [1, 1, 1, 1, 1]), None, 1, 0)
    assert out.to_vector() == [1.0, 3.0, 2.0, 4.0, 5.0, 7.0, 6.0, 8.0]


def test_gradients_accumulate_when_a_tensor_is_used_twice():
    a, b = _t([2.0], [1], True), _t([3.0], [1], True)
    lt.Ops.add(lt.Ops.add(a, b), a).backward()
    assert a.grad.item() == 2.0 and b.grad.item() == 1.0


# ---- tests/llm_optimization_test.cpp
class _Mock(lt.nn.Module):
    """Logits that depend on the position only (the reference test's MockModel)."""

    def __init__(self, rows):
        super().__init__()
        self.rows = rows

    def forward(self, x):
        import torch
        T = x.shape[1]
        return lt.Tensor(torch.tensor([[self.rows[min(s, len(self.rows) - 1)] for s in range(T)]], dtype=torch.float32))


def test_prefix_cache_hit_and_miss():
    cache = lt.nn.PrefixCache.get()
    cache.clear()
    cache.put([101, 102, 103], [_t([1.0, 2.0], [1, 2])])
    got = cache.get_cache([101, 102, 103])
    assert len(got) == 1 and got[0].to_vector()[0] == 1.0
    assert len(cache.get_cache([101, 102, 104])) == 0
    cache.clear()


def test_speculative_decoding_accepts_agreeing_drafts():
    rows = [[0.1, 0.8, 0.1], [0.1, 0.1, 0.8], [0.8, 0.1, 0.1], [0.1, 0.8, 0.1], [0.1, 0.1, 0.8]]
    eng = lt.nn.SpeculativeEngine(_Mock(rows), _Mock(rows))
    toks = eng.generate([0], 3, 2)
    assert len(toks) == 4 and toks[1] == 1 and toks[2] == 2


def test_flash_decoding_equals_flash_attention():
    q = _t([0.1, 0.2, 0.3, 0.4], [1, 1, 1, 4])
    k = _t([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8], [1, 1, 2, 4])
    v = _t([1, 2, 3, 4, 5, 6, 7, 8], [1, 1, 2, 4])
    dec, att = lt.Ops.flash_decoding(q, k, v, 2).to_vector(), lt.Ops.flash_attention(q, k, v).to_vector()
    assert all(abs(a - b) < 1e-4 for a, b in zip(dec, att))


def test_nf4_cast_round_trip():
    x = _t([0.0, -0.6, 0.5, 1.0, -1.0], [1, 5]).cast(lt.DataType.NF4)
    assert x.dtype == lt.DataType.NF4
    back = x.cast(lt.DataType.FP32).to_vector()
    assert back[0] == 0.0 and back[4] == -1.0 and abs(back[1] + 0.6961917) < 0.25


def test_qlora_linear_trains_its_adapters():
    lin = lt.nn.QLoRALinear(4, 2, 2, 16.0, True)
    out = lin.forward(_t([1, 2, 3, 4], [1, 4], True))
    assert out.shape == [1, 2]
    lt.Ops.sum(out).backward()
    assert lin.lora_A.grad is not None and lin.lora_B.grad is not None


def test_fused_linear_cross_entropy_equals_the_two_step_form():
    x, w = _t([1.0, 2.0, 0.5, -0.5], [2, 2], True), _t([0.1, 0.2, -0.3, 0.4], [2, 2], True)
    tgt = _t([0.0, 1.0], [2])
    fused = lt.Ops.fused_linear_cross_entropy(x, w, tgt)
    fused.backward()
    gx = x.grad.to_vector()
    x2, w2 = _t([1.0, 2.0, 0.5, -0.5], [2, 2], True), _t([0.1, 0.2, -0.3, 0.4], [2, 2], True)
    plain = lt.Ops.cross_entropy_loss(lt.Ops.matmul(x2, w2.transpose(0, 1)), tgt)
    plain.backward()
    assert abs(fused.to_vector()[0] - plain.to_vector()[0]) < 1e-5
    assert all(abs(a - b) < 1e-4 for a, b in zip(gx, x2.grad.to_vector()))


# ---- tests/advanced_optimization_stage2_test.cpp
def test_guided_decoding_masks():
    dec = lt.nn.GuidedDecoder(["123", "abc", "789", "xyz"])
    logits = _t([1.0, 2.0, 3.0, 4.0], [4])
    dec.apply_mask(logits, "", "digits")
    assert logits.to_vector() == [1.0, -1e9, 3.0, -1e9]
    logits2 = _t([1.0, 2.0, 3.0, 4.0], [4])
    dec.apply_mask(logits2, "", "prefix:abc")
    assert logits2.to_vector() == [-1e9, 2.0, -1e9, -1e9]


def test_w8a8_matmul_takes_the_weight_as_out_by_in():
    x, w = _t([1.5, 2.5, -3.5, 4.5], [2, 2]), _t([0.5, -1.5, 2.0, 1.0], [2, 2])
    out = lt.Ops.w8a8_matmul(x, w, 0.5, 0.5)
    assert out.shape == [2, 2]
    val0 = (round(1.5 / 0.5) * round(0.5 / 0.5) + round(2.5 / 0.5) * round(-1.5 / 0.5)) * 0.25
    assert abs(out.to_vector()[0] - val0) < 1e-5


# ---- tests/advanced_serving_test.cpp
class _NextToken(lt.nn.Module):
    """logits favour token + 1 (mod vocab) at every position (the reference test's MockModel)."""

    def __init__(self, vocab):
        super().__init__()
        self.vocab = vocab

    def forward(self, x):
        import torch
        from litetorch_b200.core import _unwrap
        tok = _unwrap(x).long()
        return lt.Tensor(torch.nn.functional.one_hot((tok + 1) % self.vocab, self.vocab).float() * 10.0)


def test_continuous_batching_generates_the_counting_sequences():
    model = _NextToken(32)
    sched = lt.nn.ServingScheduler(10, 4, 2, 8)
    r1, r2 = lt.nn.Request(1, [1, 2, 3, 4, 5, 6], 4), lt.nn.Request(2, [10, 11], 4)
    sched.add_request(r1)
    sched.add_request(r2)
    steps = 0
    while (sched.pending_queue or sched.running_queue) and steps < 50:
        sched.step(model)
        steps += 1
    assert r1.is_finished and r2.is_finished
    assert r1.generated_tokens == [7, 8, 9, 10] and r2.generated_tokens == [12, 13, 14, 15]
    assert len(sched.free_blocks) == 10 and sched.free_blocks == 10


def test_moe_linear_routes_gradients_to_gate_and_experts():
    moe = lt.nn.MoELinear(4, 4, 3, 2)
    x = _t([1, 2, 3, 4, 5, 6, 7, 8], [2, 4], True)
    out = moe.forward(x)
    assert out.shape == [2, 4]
    lt.Ops.sum(out).backward()
    assert x.grad is not None and moe.gate_weight.grad is not None
    assert any(abs(g) > 1e-5 for g in moe.gate_weight.grad.to_vector())
    assert len(moe.experts) == 3 and moe.num_experts == 3 and moe.top_k == 2


def test_medusa_heads_speed_up_the_counting_model():
    import torch
    from litetorch_b200.core import _unwrap
    base = _NextToken(32)
    heads = []
    for h in range(2):
        head = lt.nn.MedusaHead(32, 32)
        w = torch.zeros(32, 32)
        for cur in range(32):
            w[(cur + h + 2) % 32, cur] = 10.0
        with torch.no_grad():
            _unwrap(head.weight).copy_(w)
            if head.bias is not None:
                _unwrap(head.bias).zero_()
        heads.append(head)
    toks = lt.nn.MedusaEngine(base, heads).generate([1, 2], 6, 2)
    assert len(toks) >= 8 and toks[2:5] == [3, 4, 5]


# ---- tests/production_optimization_test.cpp
def test_adamw8bit_tracks_adamw_on_the_first_step():
    p1, p2 = _t([1, 2, 3], [1, 3], True), _t([1, 2, 3], [1, 3], True)
    p1.grad, p2.grad = _t([0.1, -0.2, 0.3], [1, 3]), _t([0.1, -0.2, 0.3], [1, 3])
    lt.optim.AdamW([p1], 0.1, 0.9, 0.999, 1e-8, 0.01).step()
    lt.optim.AdamW8bit([p2], 0.1, 0.9, 0.999, 1e-8, 0.01).step()
    assert all(abs(a - b) <= 0.05 for a, b in zip(p1.to_vector(), p2.to_vector()))
    assert p1.to_vector() != [1.0, 2.0, 3.0]


def test_paged_attention_of_constant_values_returns_the_value():
    import torch
    S, H, Hkv, D, bs = 2, 4, 2, 8, 4
    q = lt.Tensor(torch.full((S, H, D), 0.1))
    kc, vc = lt.Tensor(torch.full((4, Hkv, bs, D), 0.2)), lt.Tensor(torch.full((4, Hkv, bs, D), 0.3))
    bt = lt.Tensor(torch.tensor([[0, 1], [2, 3]], dtype=torch.float32))
    cl = lt.Tensor(torch.tensor([6, 8], dtype=torch.float32))
    out = lt.Ops.paged_attention(q, kc, vc, bt, cl, bs)
    assert out.shape == [S, H, D] and all(abs(v - 0.3) < 1e-4 for v in out.to_vector())


def test_custom_operator_with_the_reference_conventions():
    import torch
    from litetorch_b200.core import _unwrap
    reg = lt.custom_ops.Registry.get()
    reg.register_op("mul_by_two", lambda args: lt.Tensor(_unwrap(args[0]) * 2.0), None,
                    lambda grad_out, inputs, output: [lt.Tensor(_unwrap(grad_out) * 2.0)])
    x = _t([1, 2, 3], [1, 3], True)
    y = reg.call("mul_by_two", [x])
    assert y.to_vector() == [2.0, 4.0, 6.0]
    y.backward(_t([1, 1, 1], [1, 3]))
    assert x.grad.to_vector() == [2.0, 2.0, 2.0]
    reg.unregister("mul_by_two")


# ---- tests/production_features_test.cpp
def test_casts_round_trip_with_the_expected_values():
    D = lt.DataType
    t = _t([1.5, -2.5, 0.0, 10.25], [4])
    h = t.cast(D.FP16)
    assert h.dtype == D.FP16
    back = h.cast(D.FP32)
    assert back.dtype == D.FP32 and all(abs(a - b) < 1e-3 for a, b in zip(back.to_vector(), [1.5, -2.5, 0.0, 10.25]))
    i8 = t.cast(D.INT8)
    assert i8.dtype == D.INT8 and i8.cast(D.FP32).to_vector() == [1.0, -2.0, 0.0, 10.0]
    f64 = t.cast(D.FP64)
    assert f64.dtype == D.FP64 and abs(f64.cast(D.FP32).to_vector()[0] - 1.5) < 1e-5
    i16 = t.cast(D.INT16)
    assert i16.dtype == D.INT16 and i16.cast(D.FP32).to_vector()[0] == 1.0
    i4 = t.cast(D.INT4)
    assert i4.dtype == D.INT4 and i4.cast(D.FP32).to_vector()[0] == 1.0
    bf = t.cast(D.BF16)
    assert bf.dtype == D.BF16 and abs(bf.cast(D.FP32).to_vector()[0] - 1.5) < 1e-2


def test_half_precision_matmul_with_a_grad_scaler_moves_the_weight():
    x, w = _t([1.0, 2.0], [1, 2], True), _t([0.5, -0.5, 1.0, 2.0], [2, 2], True)
    out = lt.Ops.cast(lt.Ops.matmul(lt.Ops.cast(x, lt.DataType.FP16), lt.Ops.cast(w, lt.DataType.FP16).transpose(0, 1)), lt.DataType.FP32)
    loss = lt.Ops.mse_loss(out, _t([0.5, 4.5], [1, 2]))
    scaler = lt.amp.GradScaler(1024.0)
    scaler.scale(loss).backward()
    opt = lt.optim.SGD([x, w], 0.1)
    old = w.to_vector()[0]
    scaler.step(opt)
    scaler.update()
    assert w.to_vector()[0] != old


def test_fsdp_wrapper_flattens_and_restores_the_weight_shape():
    lin = lt.nn.Linear(4, 4, False)
    fsdp = lt.distributed.FullyShardedDataParallel(lin)
    assert lin.weight.shape[0] == 16
    fsdp.gather_parameters()
    assert lin.weight.shape == [4, 4]
    fsdp.shard_parameters()
    assert lin.weight.shape[0] == 16


def test_quantize_linear_and_calibrator_scale():
    import torch
    from litetorch_b200.core import _unwrap
    W = [0.5, -0.2, 0.8, -0.1, 1.2, 0.0, -0.5, 0.3, -0.9, 0.4, 0.1, -0.2, 0.6, -0.7, 0.3, 0.5]
    lin = lt.nn.Linear(4, 4, False)
    with torch.no_grad():
        _unwrap(lin.weight).copy_(torch.tensor(W).view(4, 4))
    lt.quantization.quantize_linear(lin)
    assert lin.weight.dtype == lt.DataType.INT8 and lin.scales is not None and lin.scales.shape[0] == 4
    assert len(lin.forward(_t([1, 1, 1, 1], [1, 4])).to_vector()) == 4
    cal = lt.quantization.Calibrator()
    cal.collect("layer1_act", _t([-2.5, 1.0, 3.2, -0.5], [1, 4]))
    assert abs(cal.get_scale("layer1_act", 8) - 3.2 / 127.0) < 1e-5
    lin2 = lt.nn.Linear(4, 4, False)
    with torch.no_grad():
        _unwrap(lin2.weight).copy_(torch.tensor(W).view(4, 4))
    # positional arguments as the reference's C++ test passes them: (linear, w_scale, w_zp, a_scale ...) - here by keyword
    qat = lt.quantization.QATLinear(lin2, w_scale=0.01, a_scale=0.01, b=8)
    qat.qat_enabled = True
    qat.train()
    x = _t([1, 2, 3, 4], [1, 4], True)
    out = qat.forward(x)
    assert out.requires_grad
    lt.Ops.sum(out).backward()
    assert x.grad is not None and qat.weight.grad is not None


# ---- tests/scale_upgrade_test.cpp
def test_fp8_casts_are_one_byte_and_round_trip():
    D = lt.DataType
    x = _t([1.0, -0.5, 2.5, 0.0, 15.0], [1, 5])
    for dt, tol in ((D.FP8_E4M3, 0.2), (D.FP8_E5M2, 0.5)):
        q = x.cast(dt)
        assert q.dtype == dt and q.element_size() == 1
        v = q.cast(D.FP32).to_vector()
        assert abs(v[0] - 1.0) < 0.1 and abs(v[1] + 0.5) < 0.1 and abs(v[2] - 2.5) < tol and v[3] == 0.0


def test_scaled_matmul_applies_both_scales():
    out = lt.Ops.scaled_matmul(_t([1, 2, 3, 4], [2, 2]), _t([1, 0, 0, 1], [2, 2]), 0.5, 2.0)
    assert all(abs(a - b) < 1e-5 for a, b in zip(out.to_vector(), [1.0, 2.0, 3.0, 4.0]))


def test_ring_attention_of_constant_values_returns_the_value():
    q, k, v = (_t([c] * 32, [1, 2, 4, 4]) for c in (0.1, 0.2, 0.3))
    out = lt.Ops.ring_attention(q, k, v, None)
    assert all(abs(x - 0.3) < 1e-4 for x in out.to_vector())


def test_adamw_fp8_steps_against_the_gradient_and_keeps_fp8_moments():
    p = _t([1.0, 2.0, 3.0], [1, 3], True)
    p.grad = _t([0.1, -0.2, 0.3], [1, 3])
    opt = lt.optim.AdamWFP8([p], 0.1, 0.9, 0.999, 1e-8, 0.01)
    opt.step()
    v = p.to_vector()
    assert v[0] < 1.0 and v[1] > 2.0 and v[2] < 3.0
    assert opt.m[0].dtype == lt.DataType.FP8_E4M3 and opt.v[0].dtype == lt.DataType.FP8_E4M3


# ---- tests/advanced_features_test.cpp
def test_meta_tensor_has_a_shape_and_no_data():
    import pytest
    t = lt.Tensor.create([2, 3, 4], lt.Device(lt.DeviceType.META, 0))
    assert t.shape == [2, 3, 4] and t.device.type == lt.DeviceType.META
    with pytest.raises(RuntimeError):
        t.data_ptr()


def test_tensor_backward_hook_scales_the_gradient():
    x = _t([1.0, 2.0], [2], True)
    y = lt.Ops.mul(x, _t([3.0, 4.0], [2]))
    x.register_hook(lambda g: lt.Ops.mul(g, _t([2.0, 2.0], [2])))
    lt.Ops.sum(y).backward()
    g = x.grad.to_vector()
    assert abs(g[0] - 6.0) < 1e-4 and abs(g[1] - 8.0) < 1e-4


def test_module_forward_hooks_run_around_the_call():
    class Double(lt.nn.Module):
        def forward(self, input):
            return lt.Ops.mul(input, _t([2.0], [1]))

    m, ran = Double(), []
    m.register_forward_pre_hook(lambda mod, inp: ran.append("pre"))
    m.register_forward_hook(lambda mod, inp, out: ran.append("post"))
    y = m(_t([1.0, 2.0], [2])).to_vector()
    assert ran == ["pre", "post"] and abs(y[0] - 2.0) < 1e-4 and abs(y[1] - 4.0) < 1e-4


def test_adamw_step_and_its_offloaded_form_lower_the_weights():
    for offload in (False, True):
        p = _t([1.0, 2.0], [2], True)
        p.grad = _t([0.1, 0.2], [2])
        lt.optim.AdamW([p], 1e-1, 0.9, 0.999, 1e-8, 0.01, offload).step()
        v = p.to_vector()
        assert v[0] < 1.0 and v[1] < 2.0


def test_cosine_annealing_reaches_the_floor_after_t_max_steps():
    p = _t([1.0], [1], True)
    opt = lt.optim.AdamW([p], 1.0)
    sched = lt.optim.CosineAnnealingLR(opt, 10, 0.0)
    sched.step()
    assert opt.get_lr() < 1.0
    for _ in range(9):
        sched.step()
    assert opt.get_lr() < 1e-5


def test_clip_grad_norm_returns_the_old_norm_and_rescales():
    p1, p2 = _t([1.0], [1], True), _t([1.0], [1], True)
    p1.grad, p2.grad = _t([10.0], [1]), _t([20.0], [1])
    assert lt.Ops.clip_grad_norm_([p1, p2], 5.0) > 22.0
    g1, g2 = p1.grad.to_vector()[0], p2.grad.to_vector()[0]
    assert abs((g1 * g1 + g2 * g2) ** 0.5 - 5.0) < 1e-2


def test_rope_with_unit_rotation_at_position_zero_keeps_the_first_pair():
    x = _t([1, 2, 3, 4, 5, 6, 7, 8], [1, 1, 2, 4], True)
    cos, sin = _t([1.0, 0.0, 0.5, 0.87], [2, 2]), _t([0.0, 1.0, 0.87, 0.5], [2, 2])
    y = lt.Ops.rope(x, cos, sin)
    v = y.to_vector()
    assert abs(v[0] - 1.0) < 1e-4 and abs(v[1] - 2.0) < 1e-4
    lt.Ops.sum(y).backward()
    assert len(x.grad.to_vector()) == 8


def test_grouped_query_attention_shapes_and_kv_head_gradients():
    q = _t([1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 1, 1, 0, 0, 0, 0, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1],
           [1, 4, 2, 4], True)
    eye = [1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1]
    k, v = _t(eye, [1, 2, 2, 4], True), _t(eye, [1, 2, 2, 4], True)
    out = lt.Ops.flash_attention(q, k, v)
    assert out.shape == [1, 4, 2, 4]
    lt.Ops.sum(out).backward()
    assert q.grad is not None and k.grad.shape[1] == 2 and v.grad.shape[1] == 2


# ---- tests/attention_test.cpp, checkpoint_test.cpp, double_backward_test.cpp, audit_optimizations_test.cpp
def test_multi_head_attention_forward_backward_reaches_input_and_q_projection():
    import math
    B, T, C = 2, 4, 8
    x = _t([math.sin(i) for i in range(B * T * C)], [B, T, C], True)
    mha = lt.nn.MultiHeadAttention(C, 2)
    mha.to(CPU)
    out = mha.forward(x)
    assert out.shape == [B, T, C]
    lt.Ops.sum(out).backward()
    assert sum(abs(g) for g in x.grad.to_vector()) > 0.0
    assert sum(abs(g) for g in mha.q_proj.weight.grad.to_vector()) > 0.0


def test_activation_checkpoint_of_a_function_gives_the_gradient():
    x = _t([1.0] * 16, [4, 4], True)
    out = lt.checkpoint(lambda inp: lt.Ops.add(lt.Ops.mul(inp, inp), inp), x)
    assert out is not None and out.requires_grad
    lt.Ops.sum(out).backward()
    assert x.grad is not None and abs(lt.Ops.sum(x.grad).item() - 48.0) < 1e-4      # d(x^2 + x)/dx = 3 at x = 1


def test_double_backward_gives_first_and_second_derivative():
    x = _t([3.0], [1], True)
    y = lt.Ops.mul(x, x)
    y.backward(None, True)
    assert abs(x.grad.item() - 6.0) < 1e-5
    grad = x.grad
    x.zero_grad()
    grad.backward(None)
    assert abs(x.grad.item() - 2.0) < 1e-5


def test_from_vector_takes_a_dtype():
    t8 = lt.Tensor.from_vector([10.0, 20.0, 30.0], [3], CPU, False, lt.DataType.INT8)
    assert t8.dtype == lt.DataType.INT8 and t8.to_vector() == [10.0, 20.0, 30.0]
    th = lt.Tensor.from_vector([1.5, 2.5, 3.5], [3], CPU, False, lt.DataType.FP16)
    assert th.dtype == lt.DataType.FP16 and all(abs(a - b) < 1e-3 for a, b in zip(th.to_vector(), [1.5, 2.5, 3.5]))


# ---- tests/transformer_test.cpp, tests/jit_test.cpp
def test_transformer_decoder_layer_in_both_modes():
    import math
    B, Tt, Tm, C = 2, 4, 6, 8
    tgt = _t([math.sin(i) for i in range(B * Tt * C)], [B, Tt, C], True)
    mem = _t([math.cos(i) for i in range(B * Tm * C)], [B, Tm, C], True)
    layer = lt.nn.TransformerDecoderLayer(C, 2, 16)
    layer.to(CPU)
    asum = lambda t: sum(abs(g) for g in t.to_vector())
    # the reference sums the output, whose gradient through the closing LayerNorm is zero up to rounding (its assertions
    # hold on rounding noise); a weighted sum tests the same gradient paths with a gradient that is really there
    ramp = _t([math.sin(0.7 * i) + 0.3 for i in range(B * Tt * C)], [B, Tt, C])
    out = layer.forward(tgt)
    assert out.shape == [B, Tt, C]
    lt.Ops.sum(lt.Ops.mul(out, ramp)).backward()
    assert asum(tgt.grad) > 1e-3 and asum(layer.self_attn.q_proj.weight.grad) > 1e-3
    for p in layer.parameters():
        p.grad = None
    tgt.grad = None
    out = layer.forward(tgt, mem)
    assert out.shape == [B, Tt, C]
    lt.Ops.sum(lt.Ops.mul(out, ramp)).backward()
    assert asum(tgt.grad) > 1e-3 and asum(mem.grad) > 1e-3 and asum(layer.multihead_attn.q_proj.weight.grad) > 1e-3


def test_jit_expression_and_traced_function_equal_eager():
    J = lt.jit
    a, b, c = (J.JITVar(J.OpType.INPUT, n) for n in "abc")
    fused = J.JITFunction("fused_gelu_add", J.gelu(a * b + c), [a, b, c])
    ta, tb, tc = _t([1, 2, -3, 4], [4]), _t([0.5, 1.5, 2.0, -1.0], [4]), _t([1, -1, 0, 2], [4])
    seq = lt.Ops.gelu(lt.Ops.add(lt.Ops.mul(ta, tb), tc)).to_vector()
    assert all(abs(x - y) < 1e-5 for x, y in zip(seq, fused([ta, tb, tc]).to_vector()))
    x0, x1 = _t([1, 2, 3], [3]), _t([0.5, 1.0, 2.0], [3])
    traced = J.Tracer.trace([x0, x1], lambda ins: lt.Ops.relu(lt.Ops.add(ins[0], ins[1])), "traced_relu_add")
    eager = lt.Ops.relu(lt.Ops.add(x0, x1)).to_vector()
    assert all(abs(x - y) < 1e-5 for x, y in zip(eager, traced([x0, x1]).to_vector()))


# ---- tests/new_features_test.cpp
def test_parameter_files_round_trip_and_reject_bad_shapes_magic_and_truncation(tmp_path):
    import struct
    import pytest
    w1, w2 = [1.5, -2.0, 3.1, 0.4], [0.1, 0.2, 0.3, 0.4, 0.5, 0.6]
    path = str(tmp_path / "test_model_weights.lt")
    lt.save_parameters([_t(w1, [2, 2]), _t(w2, [2, 3])], path)
    l1, l2 = lt.Tensor.create([2, 2], CPU), lt.Tensor.create([2, 3], CPU)
    lt.load_parameters([l1, l2], path)
    assert all(abs(a - b) < 1e-5 for a, b in zip(l1.to_vector() + l2.to_vector(), w1 + w2))
    with pytest.raises(RuntimeError):
        lt.load_parameters([lt.Tensor.create([3, 3], CPU), l2], path)
    bad = tmp_path / "bad_file.lt"
    bad.write_bytes(b"BADMAGIC")
    with pytest.raises(RuntimeError):
        lt.load_parameters([l1, l2], str(bad))
    short = tmp_path / "short_file.lt"
    short.write_bytes(b"LTW1" + struct.pack("<II", 2, 2) + struct.pack("<qq", 2, 2) + struct.pack("<Q", 4)
                      + struct.pack("<ff", 1.0, 2.0))
    with pytest.raises(RuntimeError):
        lt.load_parameters([l1, l2], str(short))
    # the failed loads left the tensors as they were
    assert all(abs(a - b) < 1e-5 for a, b in zip(l1.to_vector(), w1))


def test_adam_state_round_trips_with_step_count_and_rejects_other_shapes(tmp_path):
    import pytest
    p = lt.Tensor.create([2, 2], CPU, True)
    adam = lt.optim.Adam([p], 1e-3)
    p.grad = _t([0.0] * 4, [2, 2])
    adam.step()                                  # allocates the moments
    adam.step_count = 42
    md, vd = [0.5, 0.6, 0.7, 0.8], [0.01, 0.02, 0.03, 0.04]
    lt.Tensor(adam.m[0]).copy_(_t(md, [2, 2]))
    lt.Tensor(adam.v[0]).copy_(_t(vd, [2, 2]))
    path = str(tmp_path / "test_opt_state.lt")
    lt.save_optimizer_state(adam, path)
    other = lt.optim.Adam([p], 1e-3)
    lt.load_optimizer_state(other, path)
    assert other.step_count == 42
    assert all(abs(a - b) < 1e-5 for a, b in zip(lt.Tensor(other.m[0]).to_vector(), md))
    assert all(abs(a - b) < 1e-5 for a, b in zip(lt.Tensor(other.v[0]).to_vector(), vd))
    wrong = lt.optim.Adam([lt.Tensor.create([2, 3], CPU, True)], 1e-3)
    with pytest.raises(RuntimeError):
        lt.load_optimizer_state(wrong, path)


def test_bmm_forward_and_backward_against_a_float64_oracle():
    import torch
    B, M, K, N = 16, 64, 128, 64
    av = [(i % 100) / 50.0 - 1.0 for i in range(B * M * K)]
    bv = [(i % 100) / 100.0 - 0.5 for i in range(B * K * N)]
    a, b = _t(av, [B, M, K], True), _t(bv, [B, K, N], True)
    c = lt.Ops.bmm(a, b)
    c.backward(_t([0.1] * (B * M * N), [B, M, N]))
    ar = torch.tensor(av, dtype=torch.float64).view(B, M, K).requires_grad_()
    br = torch.tensor(bv, dtype=torch.float64).view(B, K, N).requires_grad_()
    cr = torch.bmm(ar, br)
    cr.backward(torch.full_like(cr, 0.1))
    err = lambda x, r: float((torch.tensor(x.to_vector(), dtype=torch.float64) - r.detach().reshape(-1)).abs().max())
    assert err(c, cr) < 1e-3 and err(a.grad, ar.grad) < 1e-3 and err(b.grad, br.grad) < 1e-3


def test_conv3d_max_pool3d_and_3d_linear_against_a_float64_oracle():
    import torch
    import torch.nn.functional as F
    err = lambda x, r: float((torch.tensor(x.to_vector(), dtype=torch.float64) - r.detach().reshape(-1)).abs().max())
    iv = [(i % 10) / 10.0 for i in range(2 * 2 * 64)]
    wv = [(i % 5) / 5.0 - 0.4 for i in range(3 * 2 * 27)]
    bv = [0.2 * i for i in range(3)]
    x, w, b = _t(iv, [2, 2, 4, 4, 4], True), _t(wv, [3, 2, 3, 3, 3], True), _t(bv, [3], True)
    out = lt.Ops.conv3d(x, w, b, 1, 1)
    out.backward(_t([0.1] * out.numel(), out.shape))
    xr, wr, br = (torch.tensor(v, dtype=torch.float64).view(s).requires_grad_()
                  for v, s in ((iv, (2, 2, 4, 4, 4)), (wv, (3, 2, 3, 3, 3)), (bv, (3,))))
    outr = F.conv3d(xr, wr, br, stride=1, padding=1)
    outr.backward(torch.full_like(outr, 0.1))
    assert max(err(out, outr), err(x.grad, xr.grad), err(w.grad, wr.grad), err(b.grad, br.grad)) < 1e-3

    pv = [(i % 20) / 10.0 for i in range(2 * 2 * 64)]
    x = _t(pv, [2, 2, 4, 4, 4], True)
    out = lt.Ops.max_pool3d(x, 2, 2, 0)
    out.backward(_t([0.5] * out.numel(), out.shape))
    xr = torch.tensor(pv, dtype=torch.float64).view(2, 2, 4, 4, 4).requires_grad_()
    outr = F.max_pool3d(xr, 2, 2, 0)
    outr.backward(torch.full_like(outr, 0.5))
    assert err(out, outr) < 1e-3 and err(x.grad, xr.grad) < 1e-3

    lv = [i / 10.0 for i in range(2 * 3 * 4)]
    x = _t(lv, [2, 3, 4], True)
    lin = lt.nn.Linear(4, 5)
    out = lin.forward(x)
    assert out.shape == [2, 3, 5]
    out.backward(_t([0.2] * out.numel(), out.shape))
    xr = torch.tensor(lv, dtype=torch.float64).view(2, 3, 4).requires_grad_()
    wr = torch.tensor(lin.weight.to_vector(), dtype=torch.float64).view(5, 4).requires_grad_()
    br = torch.tensor(lin.bias.to_vector(), dtype=torch.float64).requires_grad_()
    outr = F.linear(xr, wr, br)
    outr.backward(torch.full_like(outr, 0.2))
    assert max(err(out, outr), err(x.grad, xr.grad), err(lin.weight.grad, wr.grad), err(lin.bias.grad, br.grad)) < 1e-3


def test_integrity_fixes_batchnorm_of_one_value_views_clones_and_dataset():
    import math
    import pytest
    bn = lt.nn.BatchNorm2d(1)
    bn.to(CPU)
    x = _t([3.5], [1, 1, 1, 1], True)
    out = bn.forward(x)
    rv = bn.running_var.to_vector()[0]
    assert not math.isnan(rv) and not math.isinf(rv)
    out.backward(_t([1.0], [1, 1, 1, 1]))
    assert x.grad is not None
    xt = _t([1, 2, 3, 4, 5, 6], [2, 3], True).transpose(0, 1)
    with pytest.raises(RuntimeError):
        xt.view([6])
    xc = _t([0, 1, 2, 3, 4, 5], [2, 3]).transpose(0, 1).clone()
    assert xc.to_vector() == [0.0, 3.0, 1.0, 4.0, 2.0, 5.0] and xc.is_contiguous()
    ds = lt.data.TensorDataset(_t([1, 2, 3, 4], [4, 1]), _t([10, 20, 30, 40], [4, 1]))
    sx, sy = ds.get(2)
    assert sx.device == CPU and sy.device == CPU
    assert abs(sx.to_vector()[0] - 3.0) < 1e-5 and abs(sy.to_vector()[0] - 30.0) < 1e-5


# ---- tests/gpt_training_test.cpp, tests/memory_leak_test.cpp
def test_qat_decoder_under_autocast_jit_round_trip_and_single_rank_group(tmp_path):
    Q = lt.quantization

    class Decoder(lt.nn.Module):
        def __init__(self, d):
            super().__init__()
            mk = lambda i, o: Q.QATLinear(lt.nn.Linear(i, o, False), w_scale=0.01, a_scale=0.01, b=8)
            self.c_attn, self.c_proj, self.c_fc, self.c_proj2 = mk(d, 3 * d), mk(d, d), mk(d, 4 * d), mk(4 * d, d)
            for m in (self.c_attn, self.c_proj, self.c_fc, self.c_proj2):
                m.qat_enabled = True

        def forward(self, x):
            self.c_attn.forward(x)
            return self.c_proj2.forward(self.c_fc.forward(self.c_proj.forward(x)))

    x = _t([1.0, -0.5, 0.2, 0.8, -0.1, 0.4, -0.9, 0.3, -0.2, 0.5, 0.6, -0.7, 0.1, -0.3, 0.8, 0.2], [2, 8], True)
    with lt.amp.AutocastGuard(True, lt.DataType.FP16):
        out = Decoder(8).forward(x)
        assert out.shape == [2, 8]
        lt.Ops.sum(out).backward()
    assert x.grad is not None
    J = lt.jit
    a, b = J.JITVar(J.OpType.INPUT, "x"), J.JITVar(J.OpType.INPUT, "y")
    path = str(tmp_path / "gpt_jit_model.txt")
    J.JITFunction("gpt_fwd", J.gelu(a * b), [a, b]).save(path)
    assert len(J.JITFunction.load(path)([_t([1, 2, 3, 4], [4]), _t([0.5] * 4, [4])]).to_vector()) == 4
    pg = lt.distributed.ProcessGroup.get()
    pg.init(0, 1, "127.0.0.1", 12347)
    t = _t([2.0, 4.0], [2])
    pg.all_reduce(t)
    assert t.to_vector() == [2.0, 4.0]
    pg.shutdown()


def test_decoder_layer_training_loop_does_not_grow_the_process():
    import gc
    import resource

    def rss_mb():
        with open("/proc/self/status") as f:
            for line in f:
                if line.startswith("VmRSS:"):
                    return int(line.split()[1]) / 1024.0
        return resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024.0

    layer = lt.nn.TransformerDecoderLayer(16, 4, 32)
    layer.to(CPU)
    tv, mv = [0.5] * (4 * 8 * 16), [-0.5] * (4 * 12 * 16)

    def step():
        tgt, mem = _t(tv, [4, 8, 16], True), _t(mv, [4, 12, 16], True)
        lt.Ops.sum(layer.forward(tgt, mem)).backward()
        for p in layer.parameters():
            p.grad = None
    for _ in range(30):
        step()
    gc.collect()
    start = rss_mb()
    for _ in range(300):
        step()
    gc.collect()
    assert rss_mb() - start < 24.0


# ---- tests/stress_test.cpp
def test_deep_convnet_trains_with_finite_decreasing_loss():
    import math
    import torch
    g = torch.Generator().manual_seed(42)
    xv = (torch.randn(16 * 3 * 16 * 16, generator=g) * 0.2).tolist()
    yv = [1.0 if j == i % 10 else 0.0 for i in range(16) for j in range(10)]
    x, y = _t(xv, [16, 3, 16, 16]), _t(yv, [16, 10])
    nn = lt.nn
    model = nn.Sequential()
    for m in (nn.Conv2d(3, 8, 3, 1, 1), nn.BatchNorm2d(8), nn.ReLU(), nn.MaxPool2d(2, 2),
              nn.Conv2d(8, 16, 3, 1, 1), nn.BatchNorm2d(16), nn.ReLU(), nn.MaxPool2d(2, 2),
              nn.AdaptiveAvgPool2d(2, 2), nn.Flatten(), nn.Linear(64, 32), nn.LayerNorm([32]), nn.GELU(),
              nn.Linear(32, 10), nn.Softmax(-1)):
        model.add(m)
    model.to(CPU)
    opt = lt.optim.Adam(model.parameters(), 0.01)
    losses = []
    for _ in range(40):
        opt.zero_grad()
        loss = lt.Ops.mse_loss(model.forward(x), y)
        loss.backward()
        assert all(p.grad is not None for p in model.parameters())
        opt.step()
        losses.append(loss.item())
        assert not math.isnan(losses[-1]) and not math.isinf(losses[-1])
    assert losses[-1] < losses[0]


def test_matmul_256_matches_a_float64_product():
    import torch
    g = torch.Generator().manual_seed(1234)
    a, b = torch.rand(256, 256, generator=g) - 0.5, torch.rand(256, 256, generator=g) - 0.5
    c = lt.Ops.matmul(lt.Tensor.from_torch(a), lt.Tensor.from_torch(b))
    ref = a.double() @ b.double()
    assert float((torch.tensor(c.to_vector(), dtype=torch.float64).view(256, 256) - ref).abs().max()) < 1e-3

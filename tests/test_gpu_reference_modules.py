"""The reference's OWN modules, unchanged, running on the sm_100a kernels through the reference's selectors.

``xLSTMLarge`` (xlstm/xlstm_large/model.py) is built with ``chunkwise_kernel="chunkwise--b200"``,
``sequence_kernel="native_sequence__b200"``, ``step_kernel="b200"``; ``xLSTMBlockStack``
(xlstm/xlstm_block_stack.py) with ``backend="b200"`` in its sLSTM layers.  Nothing of this package's model mirror is
involved: the classes, their forward code and ``generate_tokens`` (xlstm/xlstm_large/generate.py:27-90) are the
reference's.  The reference package is looked up at run time (``conftest.reference_root``); every test skips with that
reason when no copy is present.

Tolerances: fp32 runs 1e-4 relative L2 and identical greedy tokens; bf16 runs 1e-2 on cell outputs and final states;
the reference's own chunkwise-vs-step check keeps its ``atol=4e-3, rtol=5e-2``.
"""
import numpy as np
import pytest
import torch

from conftest import import_reference, load_golden, rel_l2

pytestmark = pytest.mark.gpu
B200 = dict(chunkwise_kernel="chunkwise--b200", sequence_kernel="native_sequence__b200", step_kernel="b200")
NATIVE = dict(chunkwise_kernel="chunkwise--native_autograd", sequence_kernel="native_sequence__native", step_kernel="native")


@pytest.fixture(autouse=True)
def _exact_fp32_matmuls():
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = prev


def _large(cfg_kwargs, kernels, seed=None, state_dict=None, device="cuda", dtype=torch.float32):
    import_reference()
    from xlstm.xlstm_large.model import xLSTMLarge, xLSTMLargeConfig
    if seed is not None:
        torch.manual_seed(seed)
    model = xLSTMLarge(xLSTMLargeConfig(mode="inference", return_last_states=True, **cfg_kwargs, **kernels)).eval()
    if state_dict is not None:
        model.load_state_dict(state_dict, strict=True)
    return model.to(device=device, dtype=dtype)


# ------------------------------------------------------------------------------------------------ xLSTMLarge, fp32
def test_reference_xlstm_large_fp32_matches_golden_logits_states_and_tokens():
    """embedding_dim=512, 4 heads, 6 blocks, vocabulary 2048, ids (3,256), fp32: logits, the last block's state and
    the 32 greedy tokens of ``model.generate`` equal what the reference model gave with its native kernels on a CPU
    (tests/golden/make_golden_model.py)."""
    import xlstm_b200
    from xlstm_b200.large_model import LargeConfig, procedural_state_dict
    g = load_golden("model_config1")
    shape = dict(embedding_dim=512, num_heads=4, num_blocks=6, vocab_size=2048)
    model = _large(shape, B200, state_dict=procedural_state_dict(LargeConfig(**shape), 0))
    tokens = g["tokens"].cuda()
    with torch.no_grad():
        logits, state = model(tokens)
        gen, gen_state = model.generate(tokens, max_length=32)
    xlstm_b200.check_device_status()
    assert logits.shape == (3, 256, 2048) and len(state) == 6 and len(state[0]) == 3
    assert rel_l2(logits[:, -1].cpu(), g["logits_last"]) < 1e-4
    assert rel_l2(logits[:, ::37, ::16].cpu(), g["logits_sub"]) < 1e-4
    assert rel_l2(state[5][0].cpu(), g["c5"]) < 1e-4 and rel_l2(state[5][1].cpu(), g["n5"]) < 1e-4
    assert torch.allclose(state[5][2].cpu().reshape(g["m5"].shape), g["m5"], atol=1e-4)
    assert torch.equal(gen.cpu(), g["generated"])   # identical greedy tokens over the first 32 decode steps
    assert gen_state[0][0].shape == (3, 4, 64, 128)


def test_reference_chunkwise_vs_step_check_in_fp32():
    """The reference's own self-consistency test (tests/template_chunkwise_vs_recurrent.py:6-78) with the b200 names:
    embedding 256, 4 heads, 2 blocks, vocabulary 512, ids (2,256), seed 0; whole-sequence logits equal the
    token-by-token logits within atol 4e-3 / rtol 5e-2."""
    model = _large(dict(embedding_dim=256, num_heads=4, num_blocks=2, vocab_size=512), B200, seed=0)
    torch.manual_seed(0)
    x = torch.randint(0, 512, (2, 256)).cuda()
    with torch.no_grad():
        out, state = model(x)
        assert out.shape == (2, 256, 512) and len(state) == 2 and len(state[0]) == 3
        step_out, step_state = model(x[:, 0:1])
        assert step_out.shape == (2, 1, 512) and len(step_state) == 2 and len(step_state[0]) == 3
        st, outs = None, []
        for t in range(256):
            o, st = model(x[:, t:t + 1], st)
            outs.append(o)
    np.testing.assert_allclose(torch.cat(outs, 1).cpu().numpy(), out.cpu().numpy(), atol=4e-3, rtol=5e-2)


@pytest.mark.parametrize("prefill", [128, 150])
def test_reference_generate_equals_native_kernels_on_cpu(prefill):
    """``model.generate`` with a prefill of 128 and of 150 tokens (150 = 2 chunks + a remainder of 22, the case of
    tests/test_generation.py:101-139): the b200 kernels on the GPU give the tokens the same reference model gives on a
    CPU with the native kernel names (served by the CPU oracle)."""
    from test_boundary_cpu import _register_native_oracle
    import_reference()
    _register_native_oracle()
    shape = dict(embedding_dim=256, num_heads=4, num_blocks=2, vocab_size=512)
    cpu = _large(shape, NATIVE, seed=3, device="cpu")
    gpu = _large(shape, B200, state_dict=cpu.state_dict())
    x = torch.randint(0, 512, (2, prefill), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        ref_tokens, ref_state = cpu.generate(x, max_length=16)
        tokens, state = gpu.generate(x.cuda(), max_length=16)
    assert tokens.shape == (2, 16) and torch.equal(tokens.cpu(), ref_tokens)
    assert rel_l2(state[1][0].cpu(), ref_state[1][0]) < 1e-4


# ------------------------------------------------------------------------------------------------ xLSTMLarge, bf16
def test_reference_xlstm_large_bf16_runs_the_tensor_core_kernel():
    """bf16 model at the 512/4-head shape (DHQK=64, DHV=128: the tcgen05 kernel's shapes).  The cell of block 0 is
    checked in place: a forward hook records what the reference layer hands to ``mLSTMBackend`` and what comes back,
    and the CPU oracle recomputes it from the same bf16 inputs (<= 1e-2 on h and the final state).  Whole-sequence
    logits against token-by-token logits (the step kernel) stay within bf16 model noise."""
    import xlstm_b200
    from oracle import mlstm as O
    shape = dict(embedding_dim=512, num_heads=4, num_blocks=2, vocab_size=512)
    model = _large(shape, B200, seed=1, dtype=torch.bfloat16)
    seen = {}

    def hook(mod, args, kwargs, output):
        if "h" not in seen:
            seen.update({k: v.detach().float().cpu() for k, v in kwargs.items() if torch.is_tensor(v)})
            seen["h"], seen["state"] = output[0].detach().float().cpu(), [t.detach().float().cpu() for t in output[1]]
            seen["dtype"], seen["strides"] = kwargs["q"].dtype, kwargs["q"].stride()

    handle = model.backbone.blocks[0].mlstm_layer.mlstm_backend.register_forward_hook(hook, with_kwargs=True)
    x = torch.randint(0, 512, (2, 200), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        out, state = model(x)
    handle.remove()
    xlstm_b200.check_device_status()
    assert seen["dtype"] == torch.bfloat16 and seen["strides"][1] < seen["strides"][2]   # transposed views, bf16
    h_ref, st_ref = O.mlstm_inference(seen["q"], seen["k"], seen["v"], seen["i"], seen["f"])
    assert rel_l2(seen["h"], h_ref) < 1e-2
    assert rel_l2(seen["state"][0], st_ref[0]) < 1e-2 and rel_l2(seen["state"][1], st_ref[1]) < 1e-2
    with torch.no_grad():
        st, outs = None, []
        for t in range(200):
            o, st = model(x[:, t:t + 1], st)
            outs.append(o)
    steps = torch.cat(outs, 1)
    err = rel_l2(steps.float().cpu(), out.float().cpu())
    print("bf16 chunkwise-vs-step logits, relative L2:", err)
    assert err < 3e-2
    assert rel_l2(st[1][0].cpu(), state[1][0].cpu()) < 3e-2


# ------------------------------------------------------------------------------------------------ side channel
def test_packed_batch_through_the_reference_model_equals_per_document_runs():
    """``with packed_batch(cu_seqlens): model(x)``: every document of a packed row gets the logits and final states it
    gets when the unchanged model sees it alone; the state the model returns is that of each row's last document."""
    from xlstm_b200.backend_module import packed_batch
    model = _large(dict(embedding_dim=256, num_heads=4, num_blocks=2, vocab_size=512), B200, seed=5)
    S = 160
    x = torch.randint(0, 512, (2, S), generator=torch.Generator().manual_seed(6)).cuda()
    cu = [0, 50, 160, 160, 160 + 30, 160 + 97, 320]   # row 0: 50 + 110; row 1: an empty document, 30, 67, 63
    with torch.no_grad():
        with packed_batch(cu) as doc_states:
            logits, state = model(x)
        assert len(doc_states) == 2 and doc_states[0][0].shape[0] == len(cu) - 1
        flat = x.reshape(-1)
        for d, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
            if a == b:
                for layer in range(2):
                    assert float(doc_states[layer][0][d].abs().max()) == 0.0   # an empty document leaves the zero state
                continue
            lg, st = model(flat[a:b][None])
            assert rel_l2(logits.reshape(-1, 512)[a:b].cpu(), lg[0].cpu()) < 1e-4, d
            for layer in range(2):
                assert rel_l2(doc_states[layer][0][d].cpu(), st[layer][0][0].cpu()) < 1e-4
                assert rel_l2(doc_states[layer][1][d].cpu(), st[layer][1][0].cpu()) < 1e-4
        # returned state = last document of each row (documents 1 and 5)
        assert torch.equal(state[1][0][0], doc_states[1][0][1]) and torch.equal(state[1][0][1], doc_states[1][0][5])


def test_decode_slots_through_the_reference_model_equal_per_stream_steps():
    """``with decode_slots(slot): model(token, pool)``: three streams living in rows 4, 0 and 2 of a five-row state pool
    advance exactly as three separate single-stream calls do; rows 1 and 3 stay untouched and the large C state is
    updated where it lives."""
    import xlstm_b200
    from xlstm_b200.backend_module import decode_slots
    model = _large(dict(embedding_dim=256, num_heads=4, num_blocks=2, vocab_size=512), B200, seed=7)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 512, (1, n), generator=g).cuda() for n in (40, 70, 9, 64, 23)]
    with torch.no_grad():
        states = [model(p)[1] for p in prompts]
        pool = {l: tuple(torch.cat([s[l][k] for s in states]).contiguous() for k in range(3)) for l in range(2)}
        before = {l: tuple(t.clone() for t in pool[l]) for l in range(2)}
        slot = torch.tensor([4, 0, 2], dtype=torch.int64).cuda()   # the default integer type is accepted
        tok = torch.randint(0, 512, (3, 1), generator=g).cuda()
        c_ptr = pool[0][0].data_ptr()
        with decode_slots(slot):
            logits, new_pool = model(tok, pool)
        xlstm_b200.check_device_status()
        assert new_pool[0][0].data_ptr() == c_ptr   # in place
        for b, row in enumerate([4, 0, 2]):
            lg, st = model(tok[b:b + 1], {l: tuple(t[row:row + 1].clone() for t in before[l]) for l in range(2)})
            assert rel_l2(logits[b].cpu(), lg[0].cpu()) < 1e-5
            for l in range(2):
                for k in range(3):
                    assert rel_l2(new_pool[l][k][row].cpu(), st[l][k][0].cpu()) < 1e-5
        for row in (1, 3):
            for l in range(2):
                for k in range(3):
                    assert torch.equal(new_pool[l][k][row], before[l][k][row])
    with pytest.raises(ValueError):
        xlstm_b200.ops.prepare_slots([0, 0, 1], 3, 5, "cpu")   # two streams on one row
    with pytest.raises(ValueError):
        xlstm_b200.ops.prepare_slots([0, 7, 1], 3, 5, "cpu")   # beyond the pool


# ------------------------------------------------------------------------------------------------ sLSTM block stack
def _copy_cell_weights(dst_cell, src_cell, bf16_round=False):
    """The cell's two parameters are stored in a backend-specific internal layout (xlstm/blocks/slstm/cell.py:234-261):
    they travel between backends through the external layout R (NH, DH_in, 4, DH_out), bias (NH, 4, DH)."""
    with torch.no_grad():
        R = src_cell._recurrent_kernel_int2ext(src_cell._recurrent_kernel_.detach().float())
        b = src_cell._bias_int2ext(src_cell._bias_.detach().float())
        if bf16_round:
            R = R.bfloat16().float()
        dst_cell._recurrent_kernel_.copy_(dst_cell._recurrent_kernel_ext2int(R).reshape(dst_cell._recurrent_kernel_.shape))
        dst_cell._bias_.copy_(dst_cell._bias_ext2int(b).reshape(dst_cell._bias_.shape))


def _load_stack_weights(dst, src, bf16_round=False):
    """Every weight of `src` into `dst` (stacks of the same shape, possibly different cell backends)."""
    sd = {k: (v.detach().cpu().bfloat16().float() if bf16_round and v.is_floating_point() else v.detach().cpu())
          for k, v in src.state_dict().items() if "slstm_cell._" not in k}
    missing, unexpected = dst.load_state_dict(sd, strict=False)
    assert not unexpected and all("slstm_cell._" in k for k in missing), (missing, unexpected)
    for bd, bs in zip(dst.blocks, src.blocks):
        _copy_cell_weights(bd.xlstm.slstm_cell, bs.xlstm.slstm_cell, bf16_round)


def _slstm_stack(backend, dtype, source=None, num_blocks=4, embedding_dim=1024, seed=0):
    import_reference()
    from xlstm_b200.integration import install_slstm_backend
    install_slstm_backend()
    from xlstm.blocks.slstm.block import sLSTMBlockConfig
    from xlstm.blocks.slstm.layer import sLSTMLayerConfig
    from xlstm.xlstm_block_stack import xLSTMBlockStack, xLSTMBlockStackConfig
    torch.manual_seed(seed)
    name = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    cfg = xLSTMBlockStackConfig(
        slstm_block=sLSTMBlockConfig(slstm=sLSTMLayerConfig(num_heads=4, conv1d_kernel_size=4, backend=backend, dtype=name,
                                                            recurrent_weight_init="standard")),
        num_blocks=num_blocks, embedding_dim=embedding_dim, slstm_at="all")
    stack = xLSTMBlockStack(cfg)
    stack.reset_parameters()
    if source is not None:
        _load_stack_weights(stack, source)
    return stack.eval().to(device="cuda", dtype=dtype)


def _run_stack(stack, x):
    """Forward of the unchanged stack; the final (h, c, n, m) of every block's cell is taken from a forward hook on
    ``slstm_cell`` (the block discards it, xlstm/blocks/xlstm_block.py:77) together with the cell's input."""
    finals, inputs, outputs, handles = [], [], [], []
    for blk in stack.blocks:
        def hook(mod, args, output, finals=finals, inputs=inputs, outputs=outputs):
            inputs.append(args[0].detach())
            outputs.append(output[0].detach())
            finals.append(output[1].detach().float())
        handles.append(blk.xlstm.slstm_cell.register_forward_hook(hook))
    with torch.no_grad():
        y = stack(x)
    for h in handles:
        h.remove()
    return y, finals, inputs, outputs


def test_reference_block_stack_b200_backend_against_vanilla_full_size():
    """Four sLSTM blocks, embedding 1024, 4 heads, conv kernel 4, B=16, S=2048, bf16, recurrent weights initialised
    ("standard"; the default is zeros, which would leave R h out of the test).  The unchanged ``xLSTMBlockStack`` runs
    with backend "b200" and with backend "vanilla" on the same GPU and the same weights.

    Cell level (the kernel's own error): every block's cell output and final (h, c, n, m), recomputed by the vanilla
    cell in fp32 from the very input the b200 cell saw, within 1e-2.  Stack level: outputs of the two bf16 runs and of
    a vanilla fp32 run; the vanilla bf16 backend rounds all four states to bf16 every step (src/vanilla/__init__.py:
    67-69), so its own distance to the fp32 run is reported and bounds what can be asked of the pair."""
    import xlstm_b200
    B, S, D = 16, 2048, 1024
    ref32 = _slstm_stack("vanilla", torch.float32)
    _load_stack_weights(ref32, ref32, bf16_round=True)   # bf16-representable weights, so that all three runs share them
    ours = _slstm_stack("b200", torch.bfloat16, ref32)
    van16 = _slstm_stack("vanilla", torch.bfloat16, ref32)
    x = torch.randn(B, S, D, generator=torch.Generator().manual_seed(11))
    y_b, fin_b, in_b, out_b = _run_stack(ours, x.cuda().bfloat16())
    xlstm_b200.check_device_status()
    assert torch.isfinite(y_b.float()).all()
    # ---- cell level: vanilla fp32 cell of each block on the input the b200 cell saw
    for i, blk in enumerate(ref32.blocks):
        cell = blk.xlstm.slstm_cell
        with torch.no_grad():
            o_ref, s_ref = cell(in_b[i].float())
        e_out = rel_l2(out_b[i].float().cpu(), o_ref.cpu())
        e_st = [rel_l2(fin_b[i][k].cpu(), s_ref[k].float().cpu()) for k in range(4)]
        print(f"block {i}: cell output {e_out:.2e}, final h/c/n/m {['%.2e' % e for e in e_st]}")
        assert e_out < 1e-2 and max(e_st) < 1e-2, (i, e_out, e_st)
    # ---- stack level
    y_v, fin_v, _, _ = _run_stack(van16, x.cuda().bfloat16())
    y_r, fin_r, _, _ = _run_stack(ref32, x.cuda())
    e_pair, e_ours, e_van = rel_l2(y_b.float().cpu(), y_v.float().cpu()), rel_l2(y_b.float().cpu(), y_r.cpu()), rel_l2(y_v.float().cpu(), y_r.cpu())
    print(f"stack output: b200 vs vanilla-bf16 {e_pair:.2e}; b200 vs vanilla-fp32 {e_ours:.2e}; vanilla-bf16 vs vanilla-fp32 {e_van:.2e}")
    assert e_ours < max(1e-2, 1.25 * e_van)     # at least as close to the exact run as the reference's own bf16 backend
    assert e_pair < max(1e-2, 2.0 * e_van)
    for k, name in enumerate("hcnm"):
        e = rel_l2(fin_b[3][k].cpu(), fin_r[3][k].cpu())
        ev = rel_l2(fin_v[3][k].cpu(), fin_r[3][k].cpu())
        print(f"last block final {name}: b200 vs fp32 {e:.2e}; vanilla-bf16 vs fp32 {ev:.2e}")
        assert e < max(1e-2, 1.25 * ev)


def test_reference_block_stack_trains_through_the_b200_backward_kernel():
    """A training step of the unchanged ``xLSTMBlockStack`` (two sLSTM blocks, embedding 256, 4 heads, B=4, S=96) with
    backend "b200": loss.backward() runs the backward-through-time kernel behind every cell.  Gradients of the input
    and of ALL parameters (recurrent matrices and cell biases included) against the vanilla backend in fp32 on the
    same bf16-representable weights; the vanilla backend in bf16 gives the noise level of a bf16 stack."""
    import xlstm_b200
    B, S, D = 4, 96, 256
    ref32 = _slstm_stack("vanilla", torch.float32, num_blocks=2, embedding_dim=D)
    _load_stack_weights(ref32, ref32, bf16_round=True)
    ours = _slstm_stack("b200", torch.bfloat16, ref32, num_blocks=2, embedding_dim=D)
    van16 = _slstm_stack("vanilla", torch.bfloat16, ref32, num_blocks=2, embedding_dim=D)
    g = torch.Generator().manual_seed(21)
    x = torch.randn(B, S, D, generator=g).bfloat16().float()
    w = torch.randn(B, S, D, generator=g).bfloat16().float()

    def grads(stack, dtype):
        stack.train()
        xi = x.cuda().to(dtype).requires_grad_()
        (stack(xi).float() * w.cuda()).sum().backward()
        out = {"input": xi.grad.float().cpu()}
        for name, prm in stack.named_parameters():
            if prm.grad is not None and "slstm_cell._" not in name:
                out[name] = prm.grad.float().cpu()
        # cell parameters in the external layout, which all backends share
        for i, blk in enumerate(stack.blocks):
            cell = blk.xlstm.slstm_cell
            out[f"blocks.{i}.R"] = cell._recurrent_kernel_int2ext(cell._recurrent_kernel_.grad.float()).cpu()
            out[f"blocks.{i}.bias"] = cell._bias_int2ext(cell._bias_.grad.float()).cpu()
        return out

    g_ref = grads(ref32, torch.float32)
    g_our = grads(ours, torch.bfloat16)
    xlstm_b200.check_device_status()
    g_van = grads(van16, torch.bfloat16)
    assert set(g_our) == set(g_ref)
    worst = 0.0
    for name in sorted(g_ref):
        if float(g_ref[name].norm()) == 0.0:
            continue
        e, ev = rel_l2(g_our[name], g_ref[name]), rel_l2(g_van[name], g_ref[name])
        worst = max(worst, e)
        if name == "input" or name.endswith((".R", ".bias")):
            print(f"{name}: b200 vs vanilla-fp32 {e:.2e}; vanilla-bf16 vs vanilla-fp32 {ev:.2e}")
        assert torch.isfinite(g_our[name]).all(), name
        assert e < max(3e-2, 2.0 * ev), (name, e, ev)   # parameter gradients of a bf16 stack: sums over B*S of bf16 terms
    print(f"worst parameter gradient error {worst:.2e}")


def test_fused_layer_operators_step_aside_when_gradients_are_needed():
    """With the forward-only layer operators installed (convolution, gate projections, group norm), a training step
    takes the reference's own differentiable operators around the cell and gives the gradients of the plain stack."""
    from xlstm_b200.integration import fuse_slstm_gate_projections, pack_aware_slstm_layers
    B, S, D = 2, 48, 256
    ref32 = _slstm_stack("vanilla", torch.float32, num_blocks=1, embedding_dim=D)
    _load_stack_weights(ref32, ref32, bf16_round=True)
    plain = _slstm_stack("b200", torch.bfloat16, ref32, num_blocks=1, embedding_dim=D).train()
    fused = _slstm_stack("b200", torch.bfloat16, ref32, num_blocks=1, embedding_dim=D).train()
    assert pack_aware_slstm_layers(fused) == 1 and fuse_slstm_gate_projections(fused) == 1
    x = torch.randn(B, S, D, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    grads = []
    for stack in (plain, fused):
        xi = x.clone().requires_grad_()
        stack(xi).float().square().sum().backward()
        grads.append((xi.grad.float().cpu(), {n.replace(".ref.", "."): p.grad.float().cpu() for n, p in stack.named_parameters() if p.grad is not None}))
    assert rel_l2(grads[1][0], grads[0][0]) < 1e-3
    assert set(grads[0][1]) == set(grads[1][1])
    for name in grads[0][1]:
        if float(grads[0][1][name].norm()) > 0:
            assert rel_l2(grads[1][1][name], grads[0][1][name]) < 1e-3, name
    # and without gradients the kernels run: same output as the plain stack within the operators' rounding
    with torch.no_grad():
        assert rel_l2(fused.eval()(x).float().cpu(), plain.eval()(x).float().cpu()) < 1e-2


def test_reference_slstm_cell_b200_vs_vanilla_small_with_initial_state():
    """The reference's cell-level test shape (tests/test_slstm_cell_vanilla_vs_cuda.py:12-56: hidden 64, 4 heads,
    input (1,1,256)) plus a longer batch, with and without a random initial state, R initialised."""
    import_reference()
    from xlstm_b200.integration import install_slstm_backend
    install_slstm_backend()
    from xlstm.blocks.slstm.cell import sLSTMCell, sLSTMCellConfig
    for (Bc, Sc, hidden, heads) in ((1, 1, 256, 4), (5, 33, 256, 4)):
        torch.manual_seed(42)
        van = sLSTMCell(sLSTMCellConfig(hidden_size=hidden, num_heads=heads, backend="vanilla", dtype="float32",
                                        recurrent_weight_init="standard")).cuda()
        van.reset_parameters()
        with torch.no_grad():
            for prm in van.parameters():
                prm.copy_(prm.bfloat16().float())
        ours = sLSTMCell(sLSTMCellConfig(hidden_size=hidden, num_heads=heads, backend="b200", dtype="bfloat16",
                                         recurrent_weight_init="standard")).cuda()
        _copy_cell_weights(ours, van)
        x = torch.randn(Bc, Sc, 4 * hidden).bfloat16().cuda()
        for use_state in (False, True):
            st = None
            if use_state:
                st = torch.randn(4, Bc, hidden).cuda()
                st[2] = st[2].abs() + 0.5
                st[0] = st[0].bfloat16().float()
            with torch.no_grad():
                o_ref, s_ref = van(x.float(), st)
                o, s = ours(x, None if st is None else st.bfloat16().float())
            assert o.shape == o_ref.shape == (Bc, heads, Sc, hidden // heads)
            assert rel_l2(o.float().cpu(), o_ref.cpu()) < 1e-2
            assert rel_l2(s.float().cpu(), s_ref.cpu()) < 1e-2


def test_packed_slstm_layers_equal_per_document_runs():
    """Two sLSTM blocks of the unchanged ``xLSTMBlockStack`` on a packed batch: with the pack-aware convolution in
    front of the b200 cell (``integration.pack_aware_slstm_layers`` + ``set_document_offsets``) every document comes
    out as it does when the stack sees it alone; with the reference's own convolution the first tokens of every
    document but the first of a row are wrong (its taps reach across the boundary)."""
    from xlstm_b200.integration import pack_aware_slstm_layers, set_document_offsets
    B, S, D = 2, 96, 256
    stack = _slstm_stack("b200", torch.bfloat16, num_blocks=2, embedding_dim=D, seed=3)
    leaky_stack = _slstm_stack("b200", torch.bfloat16, num_blocks=2, embedding_dim=D, seed=3)   # same weights, reference front
    x = torch.randn(B, S, D, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    cu = [0, 40, 96, 96 + 7, 96 + 7, 192]
    flat = x.reshape(1, B * S, D)
    assert pack_aware_slstm_layers(stack) == 2
    with torch.no_grad():
        alone = torch.cat([stack(flat[:, a:e]) for a, e in zip(cu[:-1], cu[1:]) if e > a], dim=1).reshape(B, S, D)
        set_document_offsets(leaky_stack, cu)    # cells only: the reference convolution still reaches across boundaries
        leaky = leaky_stack(x)
        set_document_offsets(stack, cu)
        packed = stack(x)
        set_document_offsets(stack, None)
        rows = stack(x)
    assert rel_l2(packed.float().cpu(), alone.float().cpu()) < 1e-2
    # what the blocks ADD to the residual stream (the stream itself hides most of a difference): right with the pack-aware
    # front, visibly wrong on the first tokens behind a boundary with the reference's own convolution
    add = lambda y: (y.float() - x.float()).cpu()
    assert rel_l2(add(packed), add(alone)) < 3e-2
    e_leak, e_ok = rel_l2(add(leaky)[:, 40:43], add(alone)[:, 40:43]), rel_l2(add(packed)[:, 40:43], add(alone)[:, 40:43])
    print(f"first three tokens behind a boundary, block contribution: reference convolution {e_leak:.3f}, pack-aware {e_ok:.3f}")
    assert e_ok < 2e-3 and e_leak > 1e-2   # what the kernel fixes (with the layer's small default initialisation the leak is a
    # percent-level error of the block's contribution; the fixture of the convolution alone shows it at full size)
    # without offsets the replaced front computes what the reference front computes for plain rows
    set_document_offsets(leaky_stack, None)
    with torch.no_grad():
        want = leaky_stack(x)
    assert rel_l2(rows.float().cpu(), want.float().cpu()) < 1e-2


def test_slstm_layers_with_fused_gate_projections_equal_the_layers_own():
    """The unchanged ``xLSTMBlockStack`` (two sLSTM blocks, b200 cell) before and after every layer's four headwise gate
    projections + concatenation are handed to the one-launch kernel: same parameters, same output up to the summation
    order inside the projections."""
    from xlstm_b200.integration import fuse_slstm_gate_projections
    B, S, D = 2, 200, 256
    stack = _slstm_stack("b200", torch.bfloat16, num_blocks=2, embedding_dim=D, seed=4)
    x = torch.randn(B, S, D, generator=torch.Generator().manual_seed(6)).bfloat16().cuda()
    keys = sorted(stack.state_dict().keys())
    with torch.no_grad():
        want = stack(x)
        assert fuse_slstm_gate_projections(stack) == 2
        got = stack(x)
    assert sorted(stack.state_dict().keys()) == keys
    e = rel_l2((got.float() - x.float()).cpu(), (want.float() - x.float()).cpu())   # on what the blocks add to the stream
    print(f"block contribution, fused vs the layer's own projections: {e:.2e}")
    assert e < 1e-2 and rel_l2(got.float().cpu(), want.float().cpu()) < 2e-3

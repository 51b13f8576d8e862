"""Latent fine-tune step on tiny OPT- / Llama-shaped models (random init, synthetic token ids)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("arch", ["opt-tiny", "llama-tiny"])
def test_finetune_steps_reduce_loss_and_move_codes(arch):
    from latentq_llm_b200 import finetune as ft
    from latentq_llm_b200.quant import QLinearA16W4
    model = ft.build_model(arch, "cuda", seed=7)
    swapped = ft.quantize_decoder(model, lbit=4, gbit=16)
    assert len(swapped) == (12 if arch == "opt-tiny" else 14)
    assert all(isinstance(m, QLinearA16W4) for m in swapped)
    opt, groups = ft.build_optimizer(model, lr=2e-3)
    assert len(groups[0]["params"]) == len(swapped) and len(groups[1]["params"]) > 0
    tuner = ft.LatentFineTuner(model, opt, groups, grad_accum=2)
    batches = ft.synthetic_batches(2, 4, 64, 1024, "cuda", seed=3)      # the same data every step: loss must fall
    codes0 = swapped[0].weight.data.clone()
    losses = [float(tuner.step(batches)) for _ in range(6)]
    assert all(l == l and l < 20 for l in losses), losses
    assert losses[-1] < losses[0] - 0.05, losses
    assert not torch.equal(swapped[0].weight.data, codes0)
    assert swapped[0].weight.data.dtype == torch.int8 and not swapped[0].weight.residual.init
    assert swapped[0].weight.grad is None
    st = opt.state[swapped[0].weight]
    assert st["state1"].dtype == torch.uint8 and st["step"] == 6
    # forward in eval mode still works after training (module keeps the hook: training function, no grad needed)
    with torch.no_grad():
        out = model(input_ids=batches[0][:1])
    assert torch.isfinite(out.logits.float()).all()


def test_cuda_graph_step_matches_eager_bitwise():
    """Llama-shaped tiny model (no dropout): the captured forward + backward must leave exactly the codes, residuals and
    losses of the eager loop, over several optimizer steps (the graph keeps reading the codes the optimizer rewrites)."""
    from latentq_llm_b200 import finetune as ft
    results = []
    for use_graph in (False, True):
        model = ft.build_model("llama-tiny", "cuda", seed=11)
        swapped = ft.quantize_decoder(model, lbit=4, gbit=16)
        opt, groups = ft.build_optimizer(model, lr=2e-3)
        tuner = ft.LatentFineTuner(model, opt, groups, grad_accum=2, cuda_graph=use_graph)
        batches = ft.synthetic_batches(2, 2, 64, 1024, "cuda", seed=5)
        losses = [float(tuner.step(batches)) for _ in range(4)]
        results.append((losses, [m.weight.data.clone() for m in swapped], [m.weight.residual.residual_int.clone() for m in swapped]))
    (la, ca, ra), (lb, cb, rb) = results
    assert la == lb, (la, lb)
    assert all(torch.equal(x, y) for x, y in zip(ca, cb)) and all(torch.equal(x, y) for x, y in zip(ra, rb))
    assert lb[-1] < lb[0]


def test_cuda_graph_step_with_dropout_trains():
    from latentq_llm_b200 import finetune as ft
    model = ft.build_model("opt-tiny", "cuda", seed=7)
    ft.quantize_decoder(model, lbit=4, gbit=16)
    opt, groups = ft.build_optimizer(model, lr=2e-3)
    tuner = ft.LatentFineTuner(model, opt, groups, grad_accum=2, cuda_graph=True)
    batches = ft.synthetic_batches(2, 4, 64, 1024, "cuda", seed=3)
    losses = [float(tuner.step(batches)) for _ in range(6)]
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 0.05, losses


def test_checkpoint_roundtrip_in_reference_key_layout(tmp_path):
    """Train two steps, save the decoder in the reference's A16W4 key layout (+ residual words), load it into a freshly
    built model: codes, qparams, residuals and the eval forward are identical; keys are the ones main0.py reads."""
    from safetensors.torch import load_file
    from latentq_llm_b200 import finetune as ft
    model = ft.build_model("opt-tiny", "cuda", seed=7)
    swapped = ft.quantize_decoder(model, lbit=4, gbit=16)
    opt, groups = ft.build_optimizer(model, lr=2e-3)
    tuner = ft.LatentFineTuner(model, opt, groups, grad_accum=2)
    batches = ft.synthetic_batches(2, 4, 64, 1024, "cuda", seed=3)
    for _ in range(2):
        tuner.step(batches)
    path = str(tmp_path / "decoder.safetensors")
    assert ft.save_quantized_decoder(model, path) == len(swapped)
    keys = set(load_file(path).keys())
    assert {"model.decoder.layers.0.self_attn.q_proj.qweight", "model.decoder.layers.0.self_attn.q_proj.zeros",
            "model.decoder.layers.0.self_attn.q_proj.scales", "model.decoder.layers.0.self_attn.q_proj.bias",
            "model.decoder.layers.1.fc2.qweight"} <= keys
    fresh = ft.build_model("opt-tiny", "cuda", seed=7)
    # non-quantized parameters (biases were trained, layer norms too) travel by the ordinary state dict
    loaded = ft.load_quantized_decoder(fresh, path)
    assert len(loaded) == len(swapped)
    for a, b in zip(swapped, loaded):
        assert torch.equal(a.weight.data.view(-1), b.weight.data.view(-1))
        assert torch.equal(a.scales.data, b.scales.data) and torch.equal(a.zeros.data, b.zeros.data)
        assert torch.equal(a.weight.residual.residual_int, b.weight.residual.residual_int)
        assert a.weight.residual.lock_mu == b.weight.residual.lock_mu and not b.weight.residual.init
        assert torch.equal(a.bias.data, b.bias.data)
    x = torch.randn(3, 16, 256, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        assert torch.equal(swapped[0](x), loaded[0](x))


def test_training_state_checkpoint_resumes_bit_exactly(tmp_path):
    """Four steps in one go against two steps, save, a fresh model + optimizer, load, two more steps: same losses, codes,
    residual words, dense parameters and optimizer states (eager and captured routes)."""
    from latentq_llm_b200 import finetune as ft

    def fresh(use_graph):
        model = ft.build_model("llama-tiny", "cuda", seed=11)
        swapped = ft.quantize_decoder(model, lbit=4, gbit=16)
        opt, groups = ft.build_optimizer(model, lr=2e-3)
        return model, swapped, opt, groups, ft.LatentFineTuner(model, opt, groups, grad_accum=2, cuda_graph=use_graph)

    def snapshot(swapped, opt, groups):
        out = [m.weight.data.clone() for m in swapped] + [m.weight.residual.residual_int.clone() for m in swapped]
        out += [p.data.clone() for p in groups[1]["params"]]
        for g in groups:
            for p in g["params"]:
                out += [opt.state[p][k].clone() for k in ("state1", "state2") if k in opt.state[p]]
        return out

    for use_graph in (False, True):
        batches = ft.synthetic_batches(2, 2, 64, 1024, "cuda", seed=5)
        model, swapped, opt, groups, tuner = fresh(use_graph)
        ref_losses = [float(tuner.step(batches)) for _ in range(4)]
        ref = snapshot(swapped, opt, groups)

        model, swapped, opt, groups, tuner = fresh(use_graph)
        first = [float(tuner.step(batches)) for _ in range(2)]
        path = str(tmp_path / f"state_{int(use_graph)}.safetensors")
        assert ft.save_training_state(model, opt, groups, path, step_no=tuner.step_no) > 10
        model, swapped, opt, groups, tuner = fresh(use_graph)          # same initial weights; state comes from the file
        tuner.step_no = ft.load_training_state(model, opt, groups, path)
        assert tuner.step_no == 2
        second = [float(tuner.step(batches)) for _ in range(2)]
        assert first + second == ref_losses
        got = snapshot(swapped, opt, groups)
        assert len(got) == len(ref) and all(torch.equal(a, b) for a, b in zip(got, ref))

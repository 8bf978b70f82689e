"""End-to-end parity on the reference's own CPU-sized case: an OPT-125m-architecture model
(random init, fp32, 12 decoder layers, d_model 768, FFN 3072, ReLU, vocab 50272), calibration
128 sequences x 512 token ids uniform over the vocabulary from a seed, 4-bit, group 128,
blocksize 128, percdamp 0.01, act-order off - configuration 1 at its stated size.

The GPU driver quantizes all 72 decoder linears block by block.  Checked per layer, stage by
stage:

* the Hessian the driver accumulated through its hooks (bf16 inputs, tensor cores) against one
  accumulated in fp64 from the unquantized model's activations rounded to bf16 (torch on the
  device is the checker here; the bar is 1e-3, observed 5e-6);
* the quantization against the oracle run on that same Hessian, in fp32 and - as the arbiter -
  in fp64: reconstruction error within 2 % of the fp64 oracle's for every layer; codes >= 99.5 %
  identical to the fp32 oracle's for every q/k/v/fc1 layer (48 of 72) and for the whole first
  block.

For the out_proj and fc2 layers of the deeper blocks the fp32 oracle is not a stable yardstick:
at random init their inputs are strongly correlated, the Hessians nearly singular (eigenvalue
spread ~1e5 against the damping), and the fp32 oracle itself differs from the fp64 oracle in
0.2 - 1 % of the codes.  There the GPU (whose inverse factor is within 4x of LAPACK's fp32
accuracy) must stay within twelve times the fp32 oracle's own distance from the fp64 arbiter."""
import pytest
import torch
import torch.nn as nn

from oracle import oracle_gptq as O

pytestmark = pytest.mark.gpu


def test_opt125m_architecture_end_to_end(dgq):
    transformers = pytest.importorskip("transformers")
    from distributed_gptq_b200 import DistributedGPTQuantizer, QuantizationConfig
    from distributed_gptq_b200.coordinator import DistributedConfig
    cfg = transformers.OPTConfig(vocab_size=50272, hidden_size=768, num_hidden_layers=12,
                                 ffn_dim=3072, num_attention_heads=12, max_position_embeddings=2048,
                                 word_embed_proj_dim=768, activation_function="relu")
    torch.manual_seed(0)
    model = transformers.OPTForCausalLM(cfg).float().eval()
    nseq, seqlen = 128, 512
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 50272, (nseq, seqlen), generator=g)
    names = [n for n, m in model.named_modules()
             if isinstance(m, nn.Linear) and m.weight.numel() > 1000 and "lm_head" not in n]
    assert len(names) == 72
    mods = dict(model.named_modules())
    W0 = {n: mods[n].weight.data.clone() for n in names}

    # checker: fp64 Hessians of the unquantized model, from inputs rounded to bf16 like the
    # tensor-core path takes them, accumulated by torch on the device
    model.cuda()
    H64 = {}

    def hook(name):
        def f(mod, args):
            x = args[0].detach().reshape(-1, args[0].shape[-1]).bfloat16().double()
            H64[name] = H64.get(name, 0) + x.t() @ x
        return f
    handles = [mods[n].register_forward_pre_hook(hook(n)) for n in names]
    with torch.no_grad():
        for i in range(0, nseq, 16):
            model(input_ids=ids[i:i + 16].cuda(), use_cache=False)
    for h in handles:
        h.remove()

    # GPU side, through the public driver
    qz = DistributedGPTQuantizer(QuantizationConfig(bits=4, group_size=128, blocksize=128,
                                                    percdamp=0.01, actorder=False,
                                                    calibration_samples=nseq), DistributedConfig(),
                                 calibration_batch_size=16)
    qz.keep_hessians = True
    qz.quantize_model(model, ids, layers_to_quantize=names)
    assert qz.mode_used == "block-wise" and set(qz.quantized_layers) == set(names)
    assert qz._leader["model.decoder.layers.3.self_attn.k_proj"] == \
        "model.decoder.layers.3.self_attn.q_proj" or \
        qz._leader["model.decoder.layers.3.self_attn.q_proj"] != "model.decoder.layers.3.self_attn.q_proj"

    strict, worst = 0, {"h": 0.0, "match": 1.0, "recon": 0.0, "ratio": 0.0}
    for n in names:
        Hg = qz.hessians[n]
        herr = float((Hg.double() - H64[n].cpu()).norm() / H64[n].cpu().norm())
        worst["h"] = max(worst["h"], herr)
        assert herr <= 1e-3, (n, herr)
        r32 = O.gptq_quantize(W0[n], Hg, nseq, 4, 128, 128, 0.01, False)
        r64 = O.gptq_quantize(W0[n], Hg, nseq, 4, 128, 128, 0.01, False, dtype=torch.float64)
        codes = O.unpack_f2(qz.packed[n][f"{n}.qweight"].cpu(), 4, W0[n].shape[1])
        m32 = float((codes == r32["codes"]).float().mean())
        m64 = float((codes == r64["codes"]).float().mean())
        o64 = float((r32["codes"] == r64["codes"]).float().mean())
        Q = mods[n].weight.data.float().cpu()
        r_gpu = O.recon_error(W0[n], Q, Hg)
        r_arb = O.recon_error(W0[n], r64["Q"].float(), Hg)
        assert abs(r_gpu - r_arb) <= 0.02 * r_arb, (n, r_gpu, r_arb)
        worst["recon"] = max(worst["recon"], abs(r_gpu / r_arb - 1))
        worst["match"] = min(worst["match"], m32)
        well_conditioned = not any(k in n for k in ("out_proj", "fc2")) or ".layers.0." in n
        if well_conditioned:
            assert m32 >= 0.995, (n, m32)
            # mismatches are at adjacent levels, up to groups whose zero point moved by one
            gi = r32["g_idx"].long()
            z_gpu = qz.packed[n][f"{n}.zeros"].float().cpu()
            lvl = (codes.float() - z_gpu[:, gi]) - (r32["codes"].float() - r32["zero"][:, gi])
            assert float((lvl.abs() > 1).float().mean()) <= 5e-4, n
        else:
            # the fp32 oracle's own distance from the fp64 one is 0.1-1 % here and moves from
            # run to run with the last bits of the Hessian (atomic accumulation order): floored
            ratio = (1 - m64) / max(1 - o64, 2e-3)
            worst["ratio"] = max(worst["ratio"], ratio)
            assert ratio <= 12.0, (n, m64, o64)
            assert m32 >= 0.94, (n, m32)
        strict += m32 >= 0.995
    print(f"72 layers: {strict} with >= 99.5 % of the fp32 oracle's codes; worst Hessian error "
          f"{worst['h']:.1e}, worst code match {worst['match']:.4f}, worst reconstruction-error "
          f"deviation from the fp64 oracle {worst['recon']:.4f}, worst distance ratio {worst['ratio']:.1f}")
    assert strict >= 49, strict     # measured: 50 (all q/k/v/fc1 and the first block)

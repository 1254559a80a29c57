"""Golden vectors from the reference's own PyTorch model definitions, for the parts of the forward pass that the
reference's C++ tests hold no vector for: transformer attention and SwiGLU blocks, the RMS norms (inside the blocks and
at the trunk tip, per position and spatial), nested bottleneck blocks around transformer blocks, and the SGF metadata
encoder.

What runs, all from the reference checkout (never copied): python/katago/train/model_pytorch.py builds each net
(`Model`, which uses TransformerAttentionBlock :1979, TransformerFFNBlock :2322, RMSNormMask :181, MetadataEncoder :2708),
seeded random weights are written into it, python/export_model_pytorch.py (the reference's exporter, run unmodified as
a subprocess on a checkpoint) writes the model file, and the net's fp32 CPU forward on seeded positions gives the
expected outputs.  Stored per case: the exported model file (gzip) and the outputs; positions are regenerated from
their seeds (katago_b200.modelfile.random_positions / random_meta_rows).

    KATAGO_REFERENCE=/path/to/reference python tests/golden/make_torch_golden.py

tests/test_oracle_pins.py then checks the CPU oracle, reading the stored model files, against these outputs.
"""
import copy
import gzip
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from katago_b200 import modelfile as mf  # noqa: E402

_HEADS = dict(p1_num_channels=16, g1_num_channels=16, v1_num_channels=16, sbv2_num_channels=24, num_scorebeliefs=2, v2_size=32)
_COMMON = dict(version=17, norm_kind="fixup", bnorm_epsilon=1e-4, bnorm_running_avg_momentum=0.001, initial_conv_1x1=False,
               gamma_weight_decay_center_1=True, gpool_num_channels=16)


def _tf(layers, **kw):
    blocks = []
    for i in range(layers):
        blocks += [[f"attn{i}", "attnrope"], [f"ffn{i}", "ffnsg"]]
    cfg = dict(_COMMON, **_HEADS, block_kind=blocks, activation="silu", trunk_final_rmsnorm=True)
    cfg.update(kw)
    return cfg


# name -> (model config in the reference's format, boards, board sizes, position seed, weight seed)
TORCH_CASES = {
    # plain multi-head attention, fixed-theta 2D RoPE, per-position RMSNorm tip
    "torch_tf_fixed_rope": (_tf(2, trunk_num_channels=48, mid_num_channels=48, transformer_ffn_channels=96, transformer_heads=3,
                                transformer_kv_heads=3), 5, [19, 13, 9, 19, 11], 3001, 4001),
    # grouped-query attention (6 query heads on 3 KV heads), query/key head 32 and value head 16, learnable RoPE, spatial RMSNorm tip
    "torch_tf_gqa_learnable_rope": (_tf(2, trunk_num_channels=96, mid_num_channels=96, transformer_ffn_channels=160, transformer_heads=6,
                                        transformer_kv_heads=3, attention_query_head_dim=32, attention_value_head_dim=16,
                                        learnable_rope=True, trunk_rmsnorm_spatial=True), 4, [19, 9, 13, 19], 3002, 4002),
    # nested bottleneck block whose inner stack is attention + SwiGLU FFN (exported as nested_bottleneck_block), Mish, BN-style tip
    "torch_nbt_tf": (dict(_COMMON, **_HEADS, trunk_num_channels=64, mid_num_channels=32, outermid_num_channels=32,
                          transformer_ffn_channels=64, transformer_heads=2, transformer_kv_heads=2, activation="mish",
                          block_kind=[["b0", "bottlenest2transformerropesg"], ["b1", "bottlenest2transformerropesg"]]),
                     4, [19, 13, 9, 19], 3003, 4003),
    # convolutional net with an SGF metadata encoder (human-SL nets)
    "torch_conv_meta": (dict(_COMMON, **_HEADS, version=15, trunk_num_channels=32, mid_num_channels=32, activation="mish",
                             block_kind=[["b0", "regular"], ["b1", "regulargpool"]],
                             metadata_encoder=dict(meta_encoder_version=1, internal_num_channels=32)),
                        4, [19, 13, 9, 19], 3004, 4004),
}


def case_inputs(name):
    """Seeded inputs of a case: spatial [n,19,19,22] NHWC, global [n,19], metadata rows or None."""
    cfg, n, sizes, seed, _ = TORCH_CASES[name]
    sp, gl = mf.random_positions(n, seed=seed, board_sizes=sizes)
    meta = mf.random_meta_rows(n, seed=seed + 500) if cfg.get("metadata_encoder") else None
    return sp, gl, meta


def _randomise(model, seed):
    """Seeded weights everywhere, so that no gain is 1 and no bias 0 (a fresh initialisation leaves many at those)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("rope_freqs"):
                p.copy_(torch.empty(p.shape).uniform_(-1.0, 1.0, generator=g))
            elif p.dim() >= 2 and p.shape[0] * p.shape[1] > 1 and p.numel() > max(p.shape):
                fan_in = p.numel() // p.shape[0]
                p.copy_(torch.randn(p.shape, generator=g) * (1.0 / fan_in) ** 0.5)
            elif "norm" in name and name.endswith("weight") or name.endswith("gamma"):
                base = 0.0 if name.endswith("gamma") and getattr(model, "config", {}).get("gamma_weight_decay_center_1") and p.dim() == 4 else 1.0
                p.copy_(base + torch.empty(p.shape).uniform_(-0.5, 0.5, generator=g))
            else:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)


def main():
    ref = os.environ.get("KATAGO_REFERENCE", "/root/reference")
    pydir = os.path.join(ref, "python")
    if not os.path.isdir(pydir):
        raise SystemExit("set KATAGO_REFERENCE to the reference checkout")
    sys.path.insert(0, pydir)
    import torch
    from katago.train.model_pytorch import Model
    torch.set_num_threads(4)
    for name, (cfg, n, sizes, seed, wseed) in TORCH_CASES.items():
        cfg = copy.deepcopy(cfg)
        torch.manual_seed(wseed)
        model = Model(cfg, 19)
        model.initialize()
        _randomise(model, wseed)
        model.eval()
        work = tempfile.mkdtemp(prefix="kbtorch_")
        try:
            ckpt = os.path.join(work, "model.ckpt")
            torch.save({"model": model.state_dict(), "config": cfg}, ckpt)
            r = subprocess.run([sys.executable, "export_model_pytorch.py", "-checkpoint", ckpt, "-export-dir", os.path.join(work, "out"),
                                "-model-name", name, "-filename-prefix", name], cwd=pydir, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                raise SystemExit(f"{name}: the reference exporter failed\n{r.stdout[-3000:]}")
            with open(os.path.join(work, "out", name + ".bin"), "rb") as f:
                data = f.read()
        finally:
            shutil.rmtree(work, ignore_errors=True)
        with gzip.GzipFile(os.path.join(HERE, name + ".bin.gz"), "wb", mtime=0) as f:
            f.write(data)
        sp, gl, meta = case_inputs(name)
        with torch.no_grad():
            outs = model(torch.from_numpy(np.ascontiguousarray(sp.transpose(0, 3, 1, 2))), torch.from_numpy(gl),
                         None if meta is None else torch.from_numpy(meta))[0]
        policy, value, misc, moremisc, ownership = [o.numpy().astype(np.float32) for o in outs[:5]]
        S = 19 * 19
        # the exporter writes policy channels 0 (this move) and 5 (optimistic), score values misc[0:4] + moremisc[0:2]
        pol = policy[:, [0, 5], :]
        out = dict(policy=np.ascontiguousarray(pol[:, :, :S].transpose(0, 2, 1)), policyPass=np.ascontiguousarray(pol[:, :, S]),
                   value=value, scoreValue=np.concatenate([misc[:, 0:4], moremisc[:, 0:2]], axis=1), ownership=ownership.reshape(n, S))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, len(data), "bytes of model;", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()

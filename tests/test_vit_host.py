"""ViT skeleton and the CPU whole-model oracle (no GPU)."""
import torch

from oracle.fakequant_vit import OracleViT


def test_skeleton_names_and_sizes(pkg):
    m = pkg.create_vit("deit_small", seed=0)
    names = pkg.quantised_linear_names(m)
    assert len(names) == 48 and names[:4] == ["blocks.0.attn.qkv", "blocks.0.attn.proj", "blocks.0.mlp.fc1",
                                             "blocks.0.mlp.fc2"]
    sd = m.state_dict()
    assert tuple(sd["blocks.3.attn.qkv.weight"].shape) == (1152, 384)
    assert tuple(sd["blocks.3.mlp.fc1.weight"].shape) == (1536, 384)
    assert tuple(sd["pos_embed"].shape) == (1, 197, 384) and tuple(sd["head.weight"].shape) == (1000, 384)
    n_q = sum(sd[n + ".weight"].numel() for n in names)
    assert n_q == 21_233_664                      # quantised weights of DeiT-S
    same = pkg.create_vit("deit_small", seed=0).state_dict()
    assert all(torch.equal(sd[k], same[k]) for k in sd)


def test_oracle_vit_is_deterministic_and_batch_invariant(pkg):
    m = pkg.create_vit("deit_tiny", seed=1)
    dim, heads, depth = pkg.DEIT_CONFIGS["deit_tiny"]
    o = OracleViT(m.state_dict(), dim, heads, 2, bits=4)     # two blocks keep the CPU suite short
    x = torch.randn(4, 3, 224, 224, generator=torch.Generator().manual_seed(2))
    o(x)                                                      # calibrates
    cap = {}
    y = o(x, cap)
    assert torch.equal(y, o(x))
    halves = torch.cat([o(x[:2]), o(x[2:])])
    assert torch.allclose(y, halves, atol=1e-5)
    assert set(cap) == set(o.layer_names()) and cap["blocks.1.mlp.fc2"]["x"].shape == (4 * 197, 768)
    cb = o.codebooks["blocks.0.attn.qkv"]["act_cb"]
    assert cb.shape == (16,) and (cb == 0).sum() == 1

"""Configurations of the Nupovik tests (small sizes of their own, chosen to reach every kernel route).  Model folders,
trace sessions and the error measure are shared with tests/rimidra_helpers.py."""
from oracle import nupovik_oracle as N


def config_mixed():
    """The loop starts at the first layer and holds a token-shift mixer and a latent attention (so two runs of
    each, with a cache / state per run), a gated-linear-attention layer follows; grouped routing 4 → 2."""
    return N.make_config([
        N.wkv_spec(heads=2, dim=16, mlp=N.dense_mlp(48)),
        N.latent_spec(heads=4, dim=16, vdim=24, kv_rank=32, scale=0.3,
                      mlp=N.moe_mlp(experts=8, top=2, ff=24, groups=4, keep=2)),
        N.gla_spec(heads=2, dim=16, vdim=32, tau=8.0, mlp=N.dense_mlp(40)),
    ], width=64, vocab=96, loop=(0, 2, 2), logit_scale=0.7)


def config_ones():
    """What a usual model makes > 1 is 1 here: one head everywhere, top 1, one group, tau 1, no loop, no logit
    scale; a layer without feed-forward; sizes off the multiples of 8 (CUDA-core GEMMs even in 16 bits)."""
    return N.make_config([
        N.gla_spec(heads=1, dim=8, vdim=8, tau=1.0, mlp=None),
        N.latent_spec(heads=1, dim=10, vdim=6, kv_rank=12, scale=1.0, mlp=N.moe_mlp(experts=2, top=1, ff=12)),
        N.wkv_spec(heads=1, dim=12, mlp=N.dense_mlp(20)),
    ], width=36, vocab=50, eps=1e-5)


def config_wide():
    """Shapes that the tensor-core GEMMs tile (block-diagonal latent products, grouped expert GEMMs), key size
    64 in both recurrences, value size twice the key size, a loop of one pass in the middle, an expert count
    off the 8-multiple with three groups of two, three experts per token."""
    return N.make_config([
        N.latent_spec(heads=4, dim=64, vdim=128, kv_rank=128, scale=0.12, mlp=N.dense_mlp(192)),
        N.gla_spec(heads=2, dim=64, vdim=128, tau=16.0, mlp=N.moe_mlp(experts=6, top=3, ff=64, groups=3, keep=2)),
        N.wkv_spec(heads=4, dim=64, mlp=N.moe_mlp(experts=6, top=3, ff=64, groups=3, keep=2)),
        N.latent_spec(heads=2, dim=32, vdim=64, kv_rank=64, scale=0.2, mlp=None),
    ], width=256, vocab=264, loop=(1, 3, 1), logit_scale=2.0)


def config_far():
    """Sharp attention (a scale that makes every query look at one key, wherever it is) and recurrences that
    hardly forget (with the slow-decay weights): a key hundreds of tokens back decides the logits."""
    return N.make_config([
        N.latent_spec(heads=2, dim=16, vdim=16, kv_rank=24, scale=3.0, mlp=None),
        N.wkv_spec(heads=2, dim=8, mlp=None),
        N.gla_spec(heads=2, dim=8, vdim=16, tau=64.0, mlp=N.dense_mlp(32)),
    ], width=32, vocab=64, loop=(1, 3, 2))


CONFIGS = {"mixed": config_mixed, "ones": config_ones, "wide": config_wide, "far": config_far}

# Seeds of the random checkpoints: chosen so that no routing decision of the tests' short prompts (1, 2, 13 and
# 19 tokens) is a near tie in the oracle (group or expert margins above 0.03); in 16 bits a near tie may fall
# the other way, which is no fault of the product.  Long prompts are judged by the share of rows that agree.
SEEDS = {"mixed": 22, "ones": 0, "wide": 17, "far": 3}

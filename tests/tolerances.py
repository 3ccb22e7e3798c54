"""How far the engine's logits may lie from the plain implementation's.

float32: an absolute 1e-4 on logits of order one, stated once and never widened.

bfloat16: activations carry 8 bits of mantissa through every layer, so the error grows with depth and width and is
stated relative to the spread of the logits: ``BF16_WORST_REL[name]`` is the worst ``|engine - plain| / std(plain
logits)`` that a B200 run of every replay regime (whole, last tokens one by one, changing portions, mixed with reused
pages) showed for that tiny configuration, and a test allows twice that.  A fault of the cache or of a kernel moves a
logit by a large part of the spread; rounding does not.  A greedy token may differ from the plain implementation's only
where the plain top two logits lie closer together than three times that worst error.
"""
import torch

FLOAT32_ATOL = 1e-4

# measured worst relative errors (see the docstring); a test prints its own worst so that these can be checked again.
# Each figure is the largest that one recorded run of the GPU tests (LLB_TOLERANCE_RECORD) showed under that key,
# rounded up in the third decimal.
BF16_WORST_REL = {"A": 0.014,          # replay 0.0134
                  "B": 0.017,          # replay 0.0170, long decoding 0.0136
                  "C": 0.020,          # replay 0.0196
                  "D": 0.021,          # replay 0.0200
                  "E": 0.022,          # replay 0.0212 (0.0199 before small mixed steps were described row by row)
                  # the same models with their q and k projections scaled up (sharp attention: a lost key shows, and
                  # rounding of the scores weighs more)
                  "A sharp": 0.016,    # 0.0157
                  "C sharp": 0.025,    # 0.0250
                  "D sharp": 0.053,    # every kind of span 0.0524; persistent decode 0.0191; merge through scratch 0.0111
                  "E sharp": 0.040,    # persistent decode, 17 rows: 0.0352 in one run, 0.0400 in another (its stages add
                                       # their pieces with atomics, in whatever order they arrive)
                  "toy": 0.035,        # the toy architectures of test_engine_gpu.py: routed 0.0343, norms 0.0186
                  "real": 0.033}       # two layers at the 0.5B sizes (test_real_sizes_gpu.py): 0.0323


# The same for the tiny Kudadra configurations of tests/kudadra_configs.py (weights of order 1/sqrt(in), so the
# attention is sharper and the logits wider than in the models above).
# Here the error of a row of logits is the root mean square over the row (mean taken off), which is steadier than the
# largest single logit.
KUDADRA_BF16_WORST_REL = {"P": 0.056,         # replay 0.0556, token by token 0.0321, batch 0.0292
                          "Q": 0.080,         # replay 0.0797 (a row beside one that hangs on a cancellation), batch 0.0522
                          "R": 0.074,         # batch 0.0737 (a decay of 1 forgets nothing), replay 0.0562
                          "S": 0.031,         # replay 0.0306, heavy sinks 0.0255
                          "T": 0.023,         # replay 0.0223
                          "P sharp": 0.103,   # 0.1026 in one run, 0.0686 in another
                          "Q sharp": 0.070}   # 0.0637


# The same for the tiny Bulitar configurations of tests/bulitar_configs.py (root mean square over a row, as above).
# The embedding is multiplied by a constant of the configuration (12 in V, 1 in W) and re-enters the stream at every pass
# of the loop, so the layers' rounding weighs less in V than in W.
BULITAR_BF16_WORST_REL = {"U": 0.022,         # replay 0.0218, token by token 0.0188, batch 0.0109
                          "V": 0.005,         # replay 0.0046, batch 0.0041
                          "W": 0.016,         # replay 0.0160, batch 0.0153
                          "X": 0.016,         # token by token 0.0154, replay 0.0082
                          "U sharp": 0.026,   # 0.0259
                          "V sharp": 0.006,   # 0.0053
                          "W sharp": 0.092}   # 0.0918 (a layer without a mask, scores six times as sharp, embedding scale 1)


# The same for the tiny Kuzezen configurations of tests/kuzezen_configs.py (root mean square over a row, as above).
# The widths of A, C and D (44, 32, 50) leave few terms in every norm, and a memory head's unit norm enlarges what
# rounding did to a small output; B (width 128, tensor-core sizes) stays near 2 %.
KUZEZEN_BF16_WORST_REL = {"A": 0.175,         # replay 0.0259, token by token 0.0848, batch 0.1737
                          "B": 0.025,         # replay 0.0249, batch 0.0109
                          "C": 0.08,          # token by token 0.0703
                          "D": 0.157,         # replay 0.0244, token by token 0.1562, batch 0.0472
                          "E": 0.007,         # replay 0.0061, token by token 0.0035, batch 0.0068
                          "A sharp": 0.022, "B sharp": 0.0038, "D sharp": 0.129, "E sharp": 0.003,   # 0.0219, 0.0037, 0.1281, 0.0026
                          "A memory": 0.0085, "B memory": 0.0021}                     # 0.0082, 0.0020


# The same for the tiny Fedirax configurations of tests/fedirax_configs.py (root mean square over a row, as above).
# A differential head's output is a difference of two attention maps divided by its own root mean square, so where the
# maps nearly agree the rounding of the layer's bfloat16 input is enlarged; the narrow models (A, C, D) show it most.
FEDIRAX_BF16_WORST_REL = {"A": 0.0085,         # replay 0.0073, batch 0.0071, token by token 0.0053
                          "B": 0.0030,         # replay 0.0026, batch 0.0024
                          "C": 0.025,          # replay 0.0216, batch 0.0121 (width 32, one head of 8)
                          "D": 0.0048,         # batch 0.0042, token by token 0.0042, replay 0.0037
                          "E": 0.0032,         # replay 0.0028, batch 0.0027, token by token 0.0027
                          "A sharp": 0.022, "B sharp": 0.0054, "D sharp": 0.0145,          # 0.0188, 0.0049, 0.0125 (0.0081 in another run)
                          "A sinks": 0.0080, "B sinks": 0.0036}                            # 0.0070, 0.0031


def logits_std(plain_logits) -> float:
    """Standard deviation over all logits of the given plain results (a tensor or a collection of tensors)."""
    if isinstance(plain_logits, torch.Tensor):
        return float(plain_logits.double().std())
    if isinstance(plain_logits, dict):
        plain_logits = list(plain_logits.values())
    return float(torch.cat([t.reshape(-1).double() for t in plain_logits]).std())


def atol_for(name: str, dtype: str, plain_logits) -> float:
    if dtype == "float32":
        return FLOAT32_ATOL
    return 2.0 * BF16_WORST_REL[name] * logits_std(plain_logits)


def greedy_margin_for(name: str, dtype: str, plain_logits) -> float:
    """A generated token may differ from the plain top-1 only when the plain top two are closer than this."""
    if dtype == "float32":
        return 3.0 * FLOAT32_ATOL
    return 3.0 * BF16_WORST_REL[name] * logits_std(plain_logits)


def record(label: str, worst: float, std: float) -> None:
    """Print a test's worst error and, with LLB_TOLERANCE_RECORD=<file> in the environment, append it there, so that
    one run of the GPU tests shows every figure the table above rests on."""
    import os
    line = f"{label}: worst |diff| {worst:.4e} = {worst / max(std, 1e-30):.5f} of the logits' standard deviation {std:.4f}"
    print(line)
    path = os.environ.get("LLB_TOLERANCE_RECORD")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")

"""Module-level configuration read by the layer at call time, with the names and defaults of
the reference's ``args.py`` (args.py:1-59).  A training script sets these attributes (the
reference copies its argparse namespace over them, ViT_main.py:123-125).

If the host program already has a top-level module named ``args`` (the reference's own
scripts do), ``hot_b200.quant_matmul`` reads that module instead, so the reference's entry
points drive this implementation unchanged.
"""
from collections import defaultdict

BATCH_SIZE = 0
SEED = 0
HLQ_on_base = False
HLQ_on_decompose = False

precisionScheduling = False
milestone = " "
GogiQuantBit = 0
weightQuantBit = 0
GogwQuantBit = 0
actQuantBit = 0

eps = 1e-11

quantAuto = False
quantBWDGogi = "no"  # int, stoch, nq, no
quantBWDWgt = "no"   # int, stoch, sawb, no
quantBWDGogw = "no"  # int, stoch, nq, no
quantBWDAct = "no"   # int, stoch, sawb, no

vectorPercentile = 50
transform_scheme = "gih_gwlr"

TransformGogi = False
TransformWgt = False
TransformGogw = False
TransformInput = False

layer_quant_dict = defaultdict()

# Not in the reference: name of a fixed low-rank basis to use instead of make_WHT(tokens, pct).
# "half16" = the 8 lowest-sequency rows of H_16 (r = 8 of n = 16, the setting of the reference's
# analytic cost model, utils/analysis_calculator.py:174-175).  None = follow the reference.
lowRankPreset = None

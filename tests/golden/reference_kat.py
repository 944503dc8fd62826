"""Known-answer vectors that tenmo's own test-suite holds for the hot path.

The reference is Mojo and cannot run where these fixtures were made, so there is no generating
script: every entry is a literal copied out of the named reference test (path relative to the
reference root, with line numbers), restated as plain Python data.  The oracle is pinned against
these in test_oracle_golden.py; the CUDA library is checked against the same entries in the
gpu tests.
"""

# ---- 2-D matmul: (A, B, expected C) --------------------------------------------------------------
MM2D = [
    # tests/test_mm2d.mojo:259-266 (also tests/test_attn_matmul.mojo:35-41)
    dict(name="basic", A=[[1, 2], [3, 4]], B=[[5, 6], [7, 8]], C=[[19, 22], [43, 50]]),
    # tests/test_mm2d.mojo:269-276
    dict(name="rectangular", A=[[1, 2, 3], [4, 5, 6]], B=[[7, 8], [9, 10], [11, 12]], C=[[58, 64], [139, 154]]),
    # tests/test_mm2d.mojo:302-309
    dict(name="identity", A=[[3, 4], [5, 6]], B=[[1, 0], [0, 1]], C=[[3, 4], [5, 6]]),
]

# ---- 2-D matmul on views: base array + (shape, strides, offset) ----------------------------------
MM2D_VIEWS = [
    # tests/test_mm2d.mojo:279-299: view skips the first row (offset 3)
    dict(name="offset_view_A", A_base=[1, 2, 3, 4, 5, 6, 7, 8, 9], A_shape=(2, 3), A_strides=(3, 1), A_offset=3,
         B=[[1, 0], [0, 1], [1, 1]], C=[[10, 11], [16, 17]]),
    # tests/test_mm2d.mojo:312-325: permuted view, shape (3,2) strides (1,3)
    dict(name="permuted_view_A", A_base=[1, 2, 3, 4, 5, 6], A_shape=(3, 2), A_strides=(1, 3), A_offset=0,
         B=[[1, 2], [3, 4]], C=[[13, 18], [17, 24], [21, 30]]),
]

# ---- batched matmul with gradients of sum(C): (A, B, dA, dB) -------------------------------------
MMND_GRADS = [
    # tests/test_mmnd.mojo:12-46
    dict(name="3d_basic",
         A=[[[1, 2, 3], [4, 5, 6]], [[7, 8, 9], [10, 11, 12]]],
         B=[[[1, 2], [3, 4], [5, 6]], [[7, 8], [9, 10], [11, 12]]],
         dA=[[[3, 7, 11], [3, 7, 11]], [[15, 19, 23], [15, 19, 23]]],
         dB=[[[5, 5], [7, 7], [9, 9]], [[17, 17], [19, 19], [21, 21]]]),
    # tests/test_mmnd.mojo:49-67: A (1,2,2) broadcast over B (2,2,2); dA summed over the batch
    dict(name="3d_broadcast_A",
         A=[[[1, 2], [3, 4]]],
         B=[[[2, 0], [0, 2]], [[3, 0], [0, 3]]],
         dA=[[[5, 5], [5, 5]]],
         dB=[[[4, 4], [6, 6]], [[4, 4], [6, 6]]]),
    # tests/test_mmnd.mojo:70-88: B (1,2,2) broadcast over A (2,2,2)
    dict(name="3d_broadcast_B",
         A=[[[1, 2], [3, 4]], [[5, 6], [7, 8]]],
         B=[[[2, 0], [0, 2]]],
         dA=[[[2, 2], [2, 2]], [[2, 2], [2, 2]]],
         dB=[[[16, 16], [20, 20]]]),
    # tests/test_matmul.mojo:181-243 and 439-495: (2,3) @ (1,3,4), upstream of ones
    dict(name="2d_times_3d",
         A=[[1, 2, 3], [4, 5, 6]],
         B=[[[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]]],
         C=[[[38, 44, 50, 56], [83, 98, 113, 128]]],
         dA=[[10, 26, 42], [10, 26, 42]],
         dB=[[[5, 5, 5, 5], [7, 7, 7, 7], [9, 9, 9, 9]]]),
]

# ---- all-ones shapes: C is filled with K -----------------------------------------------------------
# tests/test_attn_matmul.mojo:61-67,100-130 (shapes) and tests/test_matmul.mojo:71-105
ONES_SHAPES = [
    ((4, 3, 5), (4, 5, 2)),
    ((2, 4, 8, 16), (2, 4, 16, 8)),
    ((2, 4, 8, 8), (2, 4, 8, 16)),
    ((1, 1, 2, 3), (1, 1, 3, 2)),
    ((1, 2, 4), (4, 9)),
    ((1, 2, 4, 8), (3, 2, 8, 4)),  # tests/test_attn_matmul.mojo broadcast batch
]

# ---- shape sweep checked against the naive i-k-j loop at atol 1e-4 ---------------------------------
# tests/test_matmul_2d_verify.mojo:48-82 and tests/test_mm2d.mojo:154-171
SHAPE_SWEEP = [
    (1, 1, 1), (1, 4, 1), (1, 4, 8), (8, 4, 1), (2, 3, 4), (4, 5, 6), (7, 2, 3), (16, 12, 8), (32, 16, 32),
    (64, 32, 64), (64, 64, 128), (65, 65, 129), (127, 63, 255), (32, 128, 64), (50, 33, 77), (8, 8, 9),
    (8, 8, 33), (8, 8, 39), (8, 4, 31), (1024, 8, 16), (4, 8, 1024), (512, 128, 1024),
]

# ---- SGD: tests/test_sgd.mojo:11-111, a (2,2) parameter of ones --------------------------------------
SGD = [
    dict(name="basic", lr=0.1, momentum=0.0, wd=0.0, grads=[1.0], expect=[0.9]),
    dict(name="momentum", lr=0.1, momentum=0.9, wd=0.0, grads=[1.0, 1.0], expect=[0.9, 0.71]),
    dict(name="weight_decay", lr=0.1, momentum=0.0, wd=0.01, grads=[1.0], expect=[0.899]),
]

# ---- accuracy: tests/test_accuracy.mojo:7-104 ---------------------------------------------------------
ACCURACY = [
    dict(pred=[[0.1, 0.9], [0.8, 0.2]], target=[1, 0], correct=2),
    dict(pred=[[0.9, 0.1], [0.2, 0.8]], target=[1, 0], correct=0),
    dict(pred=[[0.1, 0.9], [0.9, 0.1], [0.3, 0.7]], target=[1, 0, 0], correct=2),
    dict(pred=[[0.1, 0.9]], target=[1], correct=1),
    dict(pred=[[0.1, 0.8, 0.1], [0.7, 0.2, 0.1]], target=[1, 0], correct=2),
    dict(pred=[[0.5, 0.5]], target=[0], correct=1),   # tie: first index wins
    dict(pred=[[0.5, 0.5]], target=[1], correct=0),
    dict(pred=[[0.1, 0.9], [0.8, 0.2], [0.9, 0.1], [0.3, 0.7], [0.6, 0.4]], target=[1, 0, 0, 0, 0], correct=4),
]

# ---- cross-entropy: tests/test_cross_entropy.mojo:978-1060 ---------------------------------------------
CE_IGNORE_LS = dict(
    logits=[[2.0, 1.0, 0.1], [0.5, 2.0, 0.3], [0.2, 0.1, 2.5]],
    targets=[0, 1, 2], ignore_index=1, label_smoothing=0.2,
    mean_loss=0.5492352,
    mean_grad=[[-0.10383275, 0.08788316, 0.015949614], [0.0, 0.0, 0.0], [0.008757681, 0.0047521815, -0.013509899]],
    sum_loss=1.0984705,
    sum_grad=[[-0.2076655, 0.17576632, 0.03189923], [0.0, 0.0, 0.0], [0.017515361, 0.009504363, -0.027019799]],
    none_loss=[0.6103632, 0.0, 0.4881073],
)
# tests/test_cross_entropy.mojo:724-742: uniform logits give -log(1/3); :1225-1241 closed form
CE_UNIFORM = dict(logits=[[1.0, 1.0, 1.0], [1.0, 1.0, 1.0]], targets=[0, 1])
CE_BASIC = dict(logits=[[2.0, 1.0, 0.5], [1.0, 2.0, 0.1]], targets=[0, 1])

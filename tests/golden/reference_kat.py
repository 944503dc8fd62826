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

# ---- softmax over the last axis: tests/test_softmax.mojo ----------------------------------------------
# Forward literals (fp32 tests, atol 1e-5): :320-330, :346-355 (CPU) and :590-600 (GPU).
SOFTMAX_FWD = [
    dict(name="cpu_1d_basic", x=[1.0, 2.0, 3.0], y=[0.09003057, 0.24472848, 0.66524094]),        # :320-330
    dict(name="cpu_1d_negative", x=[-1.0, -2.0, -3.0], y=[0.66524094, 0.24472848, 0.09003057]),  # :346-355
    dict(name="cpu_1d_uniform", x=[1.0, 1.0, 1.0, 1.0], y=[0.25, 0.25, 0.25, 0.25]),             # :332-337
]
# Inputs whose rows must each sum to 1 and stay in [0, 1] (verify_softmax_properties_*, :290-313): :339-344 (large
# values), :367-372, :385-399 / :636-660 (3-D, last axis).
SOFTMAX_ROWS_SUM_TO_ONE = [
    [[1000.0, 1001.0, 1002.0]],
    [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]],
    [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0], [7.0, 8.0, 9.0], [1.0, 2.0, 3.0]],
]
# Gradient literals of the float64 tests.  The loss there is output.mse(target) = mean((y - t)^2)
# (tensor.mojo:3101-3121), so the gradient that reaches the softmax node is 2 (y - t) / numel; "weights" entries use
# loss = sum(y * w), whose upstream gradient is w.
SOFTMAX_BWD = [
    # :40-56
    dict(name="1d_mse", x=[[0.1, 0.2, 0.3]], mse_target=[[0.0, 1.0, 0.0]],
         dx=[[0.05957773470833636, -0.1486374678358427, 0.08905973312750633]]),
    # :94-126 (axis 1 of a 2-D tensor = last axis)
    dict(name="2d_axis1_mse", x=[[1.0, 2.0], [3.0, 4.0]], mse_target=[[0.0, 1.9], [2.9, 0.0]],
         dx=[[0.14135246274290422, -0.1413524627429042], [-0.3305161770365907, 0.3305161770365907]]),
    # :162-212 (axis 2 of a (2,2,2) tensor, rows flattened)
    dict(name="3d_axis2_mse", x=[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0], [7.0, 8.0]],
         mse_target=[[1.0, 1.0], [3.0, 2.0], [3.0, 4.0], [5.0, 6.0]],
         dx=[[-0.022714436918239593, 0.0227144369182396], [-0.07186742022860364, 0.07186742022860365],
             [0.026438546392124458, -0.026438546392124486], [0.02643854639212449, -0.026438546392124406]]),
    # :228-250
    dict(name="2d_weighted_sum", x=[[0.5, 1.5], [2.5, 0.5]], weights=[[1.0, 0.0], [0.0, 1.0]],
         dx=[[0.1966119332414562, -0.19661193324145623], [-0.10499358540343878, 0.10499358540343878]]),
    # :427-434, :449-457: loss = sum(y) => gradient 0 everywhere
    dict(name="sum_gives_zero", x=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], weights=[[1.0, 1.0, 1.0], [1.0, 1.0, 1.0]],
         dx=[[0.0, 0.0, 0.0], [0.0, 0.0, 0.0]]),
]
# The whole-matrix softmax of :129-159 (axes [0, 1]) is a last-axis softmax of the flattened matrix.
SOFTMAX_BWD.append(dict(name="2d_all_axes_mse", x=[[1.0, 2.0, 3.0, 4.0]], mse_target=[[0.0, 1.9, 2.9, 0.0]],
                        dx=[[0.0064955867864787, -0.06273006370483511, -0.2712241624609286, 0.3274586393792851]]))

# ---- ReLU: tests/test_relu.mojo ---------------------------------------------------------------------------
# (x, relu(x), gradient of sum(relu(x)) = the 0/1 mask).  :9-19, :22-56, :95-100, :169-177, :179-187, :189-196
RELU = [
    dict(x=[-1.0, 0.0, 1.0, 2.0], y=[0.0, 0.0, 1.0, 2.0], mask=[0.0, 0.0, 1.0, 1.0]),
    dict(x=[[-1.0, 2.0, 0.0], [3.0, -4.0, 5.0]], y=[[0.0, 2.0, 0.0], [3.0, 0.0, 5.0]], mask=[[0.0, 1.0, 0.0], [1.0, 0.0, 1.0]]),
    dict(x=[-3.0, 0.0, 2.0, -1.0, 5.0], y=[0.0, 0.0, 2.0, 0.0, 5.0], mask=[0.0, 0.0, 1.0, 0.0, 1.0]),
    dict(x=[-1.0, 2.0, -3.0, 4.0], y=[0.0, 2.0, 0.0, 4.0], mask=[0.0, 1.0, 0.0, 1.0]),
    dict(x=[0.0, 1.0, -1.0], y=[0.0, 1.0, 0.0], mask=[0.0, 1.0, 0.0]),      # exactly 0: mask 0 (x > 0 is false)
    dict(x=[[-1.0, 2.0], [3.0, -4.0]], y=[[0.0, 2.0], [3.0, 0.0]], mask=[[0.0, 1.0], [1.0, 0.0]]),
]

# ---- Sigmoid: tests/test_sigmoid.mojo ------------------------------------------------------------------------
# Forward (atol 1e-5): :31-38, :41-46; backward of sum(y) is y (1 - y): :89-98, :101-109 (atol 1e-5)
SIGMOID = [
    dict(x=[0.0, 100.0, -100.0, 1.0, -1.0], y=[0.5, 1.0, 0.0, 0.7310586, 0.2689414]),
    dict(x=[[0.0, 1.0], [-1.0, 2.0]], y=[[0.5, 0.7310586], [0.2689414, 0.8807970]]),
    dict(x=[[0.0, 2.0], [-2.0, 0.0]], y=[[0.5, 0.8807970], [0.1192030, 0.5]]),
]

# ---- sum reductions: tests/test_sum_mean.mojo ----------------------------------------------------------------
# :99-106 sum over axis 0 (the bias-gradient reduction); :256-265 leading-axis reduction of a 3-D tensor (mean = sum/2)
SUM_AXIS0 = [
    dict(x=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], out=[5.0, 7.0, 9.0]),
    dict(x=[[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0]], out=[6.0, 8.0, 10.0, 12.0]),   # (2,2,2) viewed as (2,4): 2 * mean
]

# ---- bias-add broadcast: tests/test_broadcast.mojo:482-505 ((4,) + (3,4), loss = sum) -------------------------
ADD_BROADCAST = dict(bias=[1.0, 2.0, 3.0, 4.0], x=[[1.0] * 4, [2.0] * 4, [3.0] * 4],
                     out=[[2.0, 3.0, 4.0, 5.0], [3.0, 4.0, 5.0, 6.0], [4.0, 5.0, 6.0, 7.0]],
                     dbias=[3.0, 3.0, 3.0, 3.0])      # each bias entry receives one unit per row

# ---- matrix @ vector, vector @ matrix with gradients of sum(result): tests/test_mv.mojo, tests/test_vm.mojo ----
MV = [
    # tests/test_mv.mojo:14-45
    dict(name="mv_no_batch", M=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], v=[1.0, 2.0, 3.0], out=[14.0, 32.0],
         dM=[[1.0, 2.0, 3.0], [1.0, 2.0, 3.0]], dv=[5.0, 7.0, 9.0]),
    # tests/test_mv.mojo:84-126: M (2,2,2) @ v (2,)
    dict(name="mv_batch_M", M=[[[1.0, 2.0], [3.0, 4.0]], [[5.0, 6.0], [7.0, 8.0]]], v=[1.0, 1.0],
         out=[[3.0, 7.0], [11.0, 15.0]], dM=[[[1.0, 1.0], [1.0, 1.0]], [[1.0, 1.0], [1.0, 1.0]]], dv=[16.0, 20.0]),
]
VM = [
    # tests/test_vm.mojo:15-48
    dict(name="vm_no_batch", v=[1.0, 2.0, 3.0], M=[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], out=[22.0, 28.0],
         dv=[3.0, 7.0, 11.0], dM=[[1.0, 1.0], [2.0, 2.0], [3.0, 3.0]]),
]

# ---- Conv2d: tests/test_cnn.mojo ---------------------------------------------------------------------------------
# Forward cases as (image spec, kernel spec, bias, stride, dilation, pad) -> expected values at listed positions
# ("full" = the whole output).  "arange1" fills 1, 2, 3, ... in row-major order; a number fills with that constant.
CONV_FWD = [
    # :860-903 known values
    dict(name="known_values", x_shape=(1, 1, 3, 3), x="arange1", k=[[[[1.0, 0.0], [0.0, 1.0]]]], bias=None,
         stride=1, dilation=1, pad=0, full=[[[[6.0, 8.0], [12.0, 14.0]]]]),
    # :149-170 bias only
    dict(name="bias_only", x_shape=(1, 1, 3, 3), x=0.0, k_shape=(2, 1, 2, 2), k=0.0, bias=[5.0, 10.0],
         stride=1, dilation=1, pad=0, out_shape=(1, 2, 2, 2), channel_fill=[5.0, 10.0]),
    # :173-193 multi-channel ones: 2 channels x 2x2 = 8
    dict(name="multi_channel", x_shape=(1, 2, 4, 4), x=1.0, k_shape=(3, 2, 2, 2), k=1.0, bias=None,
         stride=1, dilation=1, pad=0, out_shape=(1, 3, 3, 3), fill=8.0),
    # :1298-1318 ones + bias 10 = 14
    dict(name="with_bias", x_shape=(1, 1, 3, 3), x=1.0, k_shape=(1, 1, 2, 2), k=1.0, bias=[10.0],
         stride=1, dilation=1, pad=0, out_shape=(1, 1, 2, 2), fill=14.0),
    # :1321-1344 three input channels: 12
    dict(name="three_in_channels", x_shape=(1, 3, 4, 4), x=1.0, k_shape=(1, 3, 2, 2), k=1.0, bias=None,
         stride=1, dilation=1, pad=0, out_shape=(1, 1, 3, 3), fill=12.0),
    # :1347-1379 three filters filled with 1, 2, 3: 4, 8, 12
    dict(name="three_filters", x_shape=(1, 1, 4, 4), x=1.0, k_shape=(3, 1, 2, 2), k="filter_index_plus_1", bias=None,
         stride=1, dilation=1, pad=0, out_shape=(1, 3, 3, 3), channel_fill=[4.0, 8.0, 12.0]),
    # :1415-1437 stride 2 on 5x5 ones
    dict(name="stride_2", x_shape=(1, 1, 5, 5), x=1.0, k_shape=(1, 1, 2, 2), k=1.0, bias=None,
         stride=2, dilation=1, pad=0, out_shape=(1, 1, 2, 2), fill=4.0),
    # :1440-1462 stride 3, 2.0 x 0.5
    dict(name="stride_3", x_shape=(1, 1, 7, 7), x=2.0, k_shape=(1, 1, 2, 2), k=0.5, bias=None,
         stride=3, dilation=1, pad=0, out_shape=(1, 1, 2, 2), fill=4.0),
    # :1591-1616 dilation 2
    dict(name="dilation_2", x_shape=(1, 1, 7, 7), x=1.0, k_shape=(1, 1, 3, 3), k=1.0, bias=None,
         stride=1, dilation=2, pad=0, out_shape=(1, 1, 3, 3), fill=9.0),
    # :1619-1643 dilation 3 (shape only in the reference; the value follows from 4 taps of 2.0 x 0.5)
    dict(name="dilation_3", x_shape=(1, 1, 9, 9), x=2.0, k_shape=(1, 1, 2, 2), k=0.5, bias=None,
         stride=1, dilation=3, pad=0, out_shape=(1, 1, 6, 6), fill=4.0),
    # :1669-1703 stride 2, dilation 2, padding 2 on 8x8 ones
    dict(name="stride_pad_dilation", x_shape=(1, 1, 8, 8), x=1.0, k_shape=(1, 1, 3, 3), k=1.0, bias=None,
         stride=2, dilation=2, pad=2,
         full=[[[[4.0, 6.0, 6.0, 4.0], [6.0, 9.0, 9.0, 6.0], [6.0, 9.0, 9.0, 6.0], [4.0, 6.0, 6.0, 4.0]]]]),
    # :1976-1994 output 1x1
    dict(name="output_1x1", x_shape=(1, 1, 3, 3), x=1.0, k_shape=(1, 1, 3, 3), k=1.0, bias=None,
         stride=1, dilation=1, pad=0, full=[[[[9.0]]]]),
    # :1650-1666, :1511-1532, :1934-1952, :1955-1973 shapes only
    dict(name="stride_and_padding", x_shape=(1, 1, 5, 5), x=1.0, k_shape=(1, 1, 3, 3), k=1.0, bias=None,
         stride=2, dilation=1, pad=1, out_shape=(1, 1, 3, 3)),
    dict(name="padding_int", x_shape=(1, 1, 3, 3), x=1.0, k_shape=(1, 1, 2, 2), k=1.0, bias=None,
         stride=1, dilation=1, pad=1, out_shape=(1, 1, 4, 4)),
    dict(name="pointwise", x_shape=(1, 3, 4, 4), x=1.0, k_shape=(2, 3, 1, 1), k=1.0, bias=None,
         stride=1, dilation=1, pad=0, out_shape=(1, 2, 4, 4), fill=3.0),
    dict(name="large_kernel", x_shape=(1, 1, 10, 10), x=1.0, k_shape=(1, 1, 7, 7), k=1.0, bias=None,
         stride=1, dilation=1, pad=0, out_shape=(1, 1, 4, 4), fill=49.0),
]
# :196-219 and :1382-1408: image b filled with b + 1, 2x2 ones kernel => 4 (b + 1)
CONV_BATCH = dict(x_shape=(4, 1, 3, 3), k_shape=(1, 1, 2, 2), expect_first=[4.0, 8.0, 12.0, 16.0])
# Backward with an upstream gradient of ones.
CONV_BWD = [
    # :1828-1852
    dict(name="backward_simple", x_shape=(1, 1, 3, 3), x=1.0, k_shape=(1, 1, 2, 2), k=1.0, bias=[0.0],
         stride=1, dilation=1, pad=0, dbias=[4.0], dx=[[[[1.0, 2.0, 1.0], [2.0, 4.0, 2.0], [1.0, 2.0, 1.0]]]],
         dk=[[[[4.0, 4.0], [4.0, 4.0]]]]),
    # :1706-1821 batch 2, 3 -> 4 channels, stride 2, padding 1, bias 0..3: every (out, in) kernel plane has the same gradient
    dict(name="all_parameters", x_shape=(2, 3, 8, 8), x=1.0, k_shape=(4, 3, 3, 3), k=1.0, bias=[0.0, 1.0, 2.0, 3.0],
         stride=2, dilation=1, pad=1, out_shape=(2, 4, 4, 4), dbias=[32.0, 32.0, 32.0, 32.0],
         dk_plane=[[18.0, 24.0, 24.0], [24.0, 32.0, 32.0], [24.0, 32.0, 32.0]]),
]

# ---- tests/test_blas.mojo: the reference's own C-ABI seam (BLASHandle.matmul over cblas_sgemm, blashandle.mojo:108-251) ----
# ta / tb: the call's transpose_A / transpose_B flags; "C" full result, "C00" the one element the reference asserts,
# "dA" / "dB" gradients of sum(C).
BLAS_SEAM = [
    # :77-91
    dict(name="simple_f32", A=[[1.0, 2.0], [3.0, 4.0]], B=[[5.0, 6.0], [7.0, 8.0]], ta=False, tb=False,
         C=[[19.0, 22.0], [43.0, 50.0]]),
    # :109-123  A @ I = A
    dict(name="identity", A=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], B=[[1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]],
         ta=False, tb=False, C=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]),
    # :126-144
    dict(name="rectangular", A=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]],
         B=[[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0], [9.0, 10.0, 11.0, 12.0]], ta=False, tb=False, shape=(2, 4), C00=38.0),
    # :150-170  A^T @ B
    dict(name="transpose_a", A=[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], B=[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], ta=True, tb=False,
         shape=(2, 2), C00=35.0),
    # :173-190  A @ B^T
    dict(name="transpose_b", A=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], B=[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], ta=False, tb=True,
         shape=(2, 2), C00=14.0),
    # :193-210  A^T @ B^T
    dict(name="transpose_both", A=[[1.0, 2.0], [3.0, 4.0]], B=[[5.0, 6.0], [7.0, 8.0]], ta=True, tb=True, shape=(2, 2), C00=23.0),
    # :258-285  gradients of sum(A @ B)
    dict(name="backward_simple", A=[[1.0, 2.0], [3.0, 4.0]], B=[[5.0, 6.0], [7.0, 8.0]], ta=False, tb=False,
         dA=[[11.0, 15.0], [11.0, 15.0]], dB=[[4.0, 4.0], [6.0, 6.0]]),
    # :640-694  gradients of sum(A^T @ B) (the values the reference prints as its expectation)
    dict(name="case_2_At_B", A=[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]],
         B=[[7.0, 8.0, 9.0], [10.0, 11.0, 12.0], [13.0, 14.0, 15.0]], ta=True, tb=False,
         dA=[[24.0, 24.0], [33.0, 33.0], [42.0, 42.0]], dB=[[3.0, 3.0, 3.0], [7.0, 7.0, 7.0], [11.0, 11.0, 11.0]]),
]
# :216-232 ones(100,100) @ ones(100,100): every element 100;  :469-486 ones(100,1) @ ones(1,100): every element 1
BLAS_SEAM_ONES = [dict(M=100, K=100, N=100, value=100.0), dict(M=100, K=1, N=100, value=1.0)]
# :1033-1088 central difference of sum(A @ B) in A[0,0] with eps 1e-4 against the analytic gradient, tolerance 0.014
BLAS_SEAM_FD = dict(A=[[1.0, 2.0], [3.0, 4.0]], B=[[5.0, 6.0], [7.0, 8.0]], eps=1e-4, tol=0.014, dA00=11.0)

# ---- tests/test_dot.mojo: vector . vector ----
DOT = [
    dict(a=[1.0, 2.0, 3.0], b=[4.0, 5.0, 6.0], value=32.0),        # :18-24, gradients :108-116 (da = b, db = a)
    dict(a=[1.0, 1.0, 1.0, 1.0], b=[2.0, 3.0, 4.0, 5.0], value=14.0),   # :27-33
    dict(a=[1.0, -2.0, 3.0], b=[-1.0, 2.0, -3.0], value=-14.0),     # :36-42
    dict(a=[3.0], b=[7.0], value=21.0),                              # :45-50
    dict(a=[1.0, 0.0], b=[0.0, 1.0], value=0.0),                     # :53-59
    dict(a=[3.0, 7.0, 2.0], b=[1.0, 1.0, 1.0], value=12.0),          # :137-145 (gradients: ones and a)
]
# :148-160  loss = d + d with d = a . b: gradients 2 b and 2 a
DOT_CHAINED = dict(a=[1.0, 2.0, 3.0], b=[4.0, 5.0, 6.0], da=[8.0, 10.0, 12.0], db=[2.0, 4.0, 6.0])

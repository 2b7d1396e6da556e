"""Known-answer vectors held by the reference's own test-suite for the PRAD Tensor / TensorReverse /
PradOp operations that this library implements, transcribed as data (inputs, expected outputs and
the decimal places the xUnit assertion compares).  Used twice: against the CPU oracle
(test_oracle_pins.py, no GPU) and against the CUDA entry points (test_gpu_reference_vectors.py).

Each case: (label, operation, inputs..., expected..., places) with places = None for Assert.Equal
on the raw doubles (exact) and an integer for DoubleArrayEqualityComparer(places) /
Assert.Equal(a, b, places).  Sources are files under test/ParallelReverseAutoDiff.Test/PRAD/.
"""
import numpy as np

PI = np.pi
A4 = [1.0, 2.0, 3.0, 4.0]
B4 = [5.0, 6.0, 7.0, 8.0]
ONES4 = [1.0, 1.0, 1.0, 1.0]
ANGLES = [0.0, PI / 2, PI, 3 * PI / 2]

# (label, op, a, b, upstream, expected_da, expected_db, places)
BINARY_REVERSE = [
    ("TensorReverseTests.cs:11-26 ElementwiseAddReverse_Test", "add", A4, B4, ONES4, ONES4, ONES4, None),
    ("TensorReverseTests.cs:29-44 ElementwiseMultiplyReverse_Test", "mul", A4, B4, ONES4, B4, A4, None),
    ("TensorReverseTests.cs:413-427 ElementwiseSubReverse_Test", "sub", A4, B4, ONES4, ONES4, [-1.0] * 4, None),
    ("TensorReverseTests.cs:430-444 ElementwiseDivideReverse_Test", "div", [2.0, 4.0, 6.0, 8.0], A4, ONES4,
     [1.0, 0.5, 1.0 / 3.0, 0.25], [-2.0, -1.0, -2.0 / 3.0, -0.5], 6),
    # PradOp.DivInto(t): t / seed; gradients[0] is the denominator's, gradients[1] the numerator's
    ("PradOpTests.cs:4086-4105 TestElementwiseDivInto", "div", [10.0, 20.0, 40.0, 80.0], [2.0, 4.0, 8.0, 16.0], ONES4,
     [0.5, 0.25, 0.125, 0.0625], [-2.5, -1.25, -0.625, -0.3125], None),
    # PradOp.SubFrom(t): t - seed
    ("PradOpTests.cs:4067-4083 TestElementwiseSubFrom", "sub", [10.0, 11.0, 12.0, 13.0], [5.0, 6.0, 7.0, 8.0], ONES4,
     ONES4, [-1.0] * 4, None),
]

# (label, op, a, b, expected, places)
BINARY_FORWARD = [
    ("PradOpTests.cs:260-275 TestElementwiseAddition", "add", A4, B4, [6.0, 8.0, 10.0, 12.0], None),
    ("PradOpTests.cs:278-293 TestElementwiseSubtraction", "sub", B4, A4, [4.0] * 4, None),
    ("PradOpTests.cs:296-311 TestElementwiseMultiplication", "mul", A4, [2.0] * 4, [2.0, 4.0, 6.0, 8.0], None),
    ("PradOpTests.cs:4067-4083 TestElementwiseSubFrom", "sub", [10.0, 11.0, 12.0, 13.0], [5.0, 6.0, 7.0, 8.0], [5.0] * 4, None),
    ("PradOpTests.cs:4086-4105 TestElementwiseDivInto", "div", [10.0, 20.0, 40.0, 80.0], [2.0, 4.0, 8.0, 16.0], [5.0] * 4, None),
]

# (label, op, x, upstream, expected_dx, places)
UNARY_REVERSE = [
    ("TensorReverseTests.cs:222-235 ElementwiseSquareReverse_Test", "square", A4, ONES4, [2.0, 4.0, 6.0, 8.0], None),
    ("TensorReverseTests.cs:238-251 ElementwiseSquareRootReverse_Test", "sqrt", [1.0, 4.0, 9.0, 16.0], ONES4,
     [0.5, 0.25, 1.0 / 6.0, 0.125], 6),
    ("TensorReverseTests.cs:254-267 ElementwiseSinReverse_Test", "sin", ANGLES, ONES4, [1.0, 0.0, -1.0, 0.0], 6),
    ("TensorReverseTests.cs:270-283 ElementwiseCosReverse_Test", "cos", ANGLES, ONES4, [0.0, -1.0, 0.0, 1.0], 6),
    ("PradOpTests.cs:314-328 TestElementwiseSin (gradient)", "sin", ANGLES, ONES4, [1.0, 0.0, -1.0, 0.0], 5),
    ("PradOpTests.cs:331-345 TestElementwiseCos (gradient)", "cos", ANGLES, ONES4, [0.0, -1.0, 0.0, 1.0], 5),
]

# (label, op, x, expected, places)
UNARY_FORWARD = [
    ("PradOpTests.cs:314-328 TestElementwiseSin", "sin", ANGLES, [0.0, 1.0, 0.0, -1.0], 5),
    ("PradOpTests.cs:331-345 TestElementwiseCos", "cos", ANGLES, [1.0, 0.0, -1.0, 0.0], 5),
]

# (label, table shape, table, indices, expected gather, upstream, expected reverse)
GATHER = [
    ("PradOpTests.cs:503-518 TestGather", (3, 2), [1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2.0, 0.0], [5.0, 6.0, 1.0, 2.0],
     [1.0] * 4, [1.0, 1.0, 0.0, 0.0, 1.0, 1.0]),
    ("TensorReverseTests.cs:101-117 GatherReverse_Test", (3, 3), [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0, 9.0], [0.0, 2.0],
     [1.0, 2.0, 3.0, 7.0, 8.0, 9.0], [1.0] * 6, [1.0, 1.0, 1.0, 0.0, 0.0, 0.0, 1.0, 1.0, 1.0]),
]

# (label, input shape, multiples, upstream (tiled shape, row-major), expected reverse)
TILE_REVERSE = [
    ("TensorReverseTests.cs:119-139 TileReverse_Test", (2, 2), (2, 2),
     [1.0, 2.0, 3.0, 4.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0, 5.0, 6.0, 7.0, 8.0], [16.0, 20.0, 16.0, 20.0]),
    ("TensorReverseTests.cs:142-160 TileReverse2_Test", (1, 4), (2, 1), [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0],
     [6.0, 8.0, 10.0, 12.0]),
    ("TensorReverseTests.cs:163-183 TileReverse3_Test", (4, 1), (1, 4),
     [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0], [10.0, 26.0, 10.0, 26.0]),
    ("PradOpTests.cs:469-483 TestTile (gradient)", (4, 1), (1, 2), [1.0] * 8, [2.0, 2.0, 2.0, 2.0]),
    ("PradOpTests.cs:486-500 TestTile2 (gradient)", (2, 2), (2, 2), [1.0] * 16, [4.0, 4.0, 4.0, 4.0]),
]

# (label, input shape, input, multiples, expected)
TILE_FORWARD = [
    ("PradOpTests.cs:469-483 TestTile", (4, 1), A4, (1, 2), [1.0, 1.0, 2.0, 2.0, 3.0, 3.0, 4.0, 4.0]),
    ("PradOpTests.cs:486-500 TestTile2", (2, 2), A4, (2, 2),
     [1.0, 2.0, 1.0, 2.0, 3.0, 4.0, 3.0, 4.0, 1.0, 2.0, 1.0, 2.0, 3.0, 4.0, 3.0, 4.0]),
]

# TensorReverseTests.cs:346-359 SumRowsReverse_Test: tensor 3x2, upstream 3x1 -> every column gets the row's value
SUM_ROWS_REVERSE = ("TensorReverseTests.cs:346-359 SumRowsReverse_Test", (3, 2), [1.0, 2.0, 3.0], [1.0, 1.0, 2.0, 2.0, 3.0, 3.0])

# TensorReverseTests.cs:362-375 TransposeReverse_Test (2-D, permutation {1,0}) and :378-410 (3-D, {0,2,1}):
# (label, original (depth, rows, cols), upstream in the transposed layout, expected)
TRANSPOSE_REVERSE = [
    ("TensorReverseTests.cs:362-375 TransposeReverse_Test", (1, 2, 3), [1.0, 4.0, 2.0, 5.0, 3.0, 6.0],
     [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]),
    ("TensorReverseTests.cs:378-410 TransposeReverse_3D_Test", (2, 3, 4),
     [1, 5, 9, 2, 6, 10, 3, 7, 11, 4, 8, 12, 13, 17, 21, 14, 18, 22, 15, 19, 23, 16, 20, 24],
     list(range(1, 25))),
]


def check(got, expected, places, label):
    got = np.asarray(got, np.float64).ravel()
    expected = np.asarray(expected, np.float64).ravel()
    assert got.shape == expected.shape, label
    if places is None:
        np.testing.assert_array_equal(got, expected, err_msg=label)
    else:   # xUnit: equal after rounding to `places` decimals
        np.testing.assert_array_equal(np.round(got, places) + 0.0, np.round(expected, places) + 0.0, err_msg=label)

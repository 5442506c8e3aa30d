"""Known-answer vectors of the reference's quantised-convolution tests, kept as
literal data.  Source: tests/test_cases/convolution_gpu_test.cpp (clDNN tree).

Each feature is (input[4], weights[3], bias, quantization, pre_relu_output[2]);
the fixture (ConvQuantizedTest::do_test, :4007-4099) builds a 1 x n x 1 x 4
input, a diagonal n x n x 1 x 3 filter, i32 bias, per-feature f32 quantisation
factors, fused ReLU, stride 1, no padding, and expects
clamp(max(0, pre_relu)) in the output type, compared exactly for integers.
"""

CASES = {
    # ConvQuantizedTest_i8_to_u8.basic, :4104-4128
    "i8_to_u8": dict(in_dtype="int8", out_dtype="uint8", features=[
        ([125, 125, 0, 1], [2, 0, 1], 1, 1.0, [251, 252]),
        ([0, 50, 0, -50], [0, 4, 4], 1, 1.0, [201, -199]),
        ([0, 50, 0, -50], [0, 8, 8], 2, 0.5, [201, -199]),
        ([120, 120, 120, -120], [1, 1, 1], 0, 0.25, [90, 30]),
        ([125, 125, 0, 126], [1, 1, 1], 1, 0.5, [126, 126]),
        ([125, 125, 0, 126], [1, 1, 1], 2, 0.5, [126, 127]),
        ([125, 125, 0, 126], [1, 1, 1], 21, 0.5, [136, 136]),
        ([0, 50, 0, -50], [0, 8, 8], 2, 1.0, [402, -398]),
    ]),
    # ConvQuantizedTest_u8_to_u8.basic, :4133-4166
    "u8_to_u8": dict(in_dtype="uint8", out_dtype="uint8", features=[
        ([125, 125, 0, 1], [2, 0, 1], 1, 1.0, [251, 252]),
        ([0, 50, 0, 50], [0, 4, -4], 1, 1.0, [201, -199]),
        ([0, 50, 0, 50], [0, 8, -8], 2, 0.5, [201, -199]),
        ([240, 240, 240, 240], [2, 1, -1], 0, 0.125, [60, 60]),
        ([125, 125, 0, 126], [1, 1, 1], 1, 0.5, [126, 126]),
        ([125, 125, 0, 126], [1, 1, 1], 2, 0.5, [126, 127]),
        ([125, 125, 0, 126], [1, 1, 1], 21, 0.5, [136, 136]),
        ([0, 50, 0, 50], [0, 8, -8], 2, 1.0, [402, -398]),
        ([250, 250, 0, 1], [1, 0, 1], 1, 1.0, [251, 252]),
        ([0, 200, 0, 200], [0, 1, -1], 1, 1.0, [201, -199]),
        ([0, 200, 0, 200], [0, 2, -2], 2, 0.5, [201, -199]),
    ]),
    # ConvQuantizedTest_u8_to_i8.basic, :4171-4182
    "u8_to_i8": dict(in_dtype="uint8", out_dtype="int8", features=[
        ([125, 125, 0, 1], [2, 0, 1], 1, 0.5, [126, 126]),
        ([125, 125, 0, 1], [2, 0, 1], 1, 1.0, [251, 252]),
        ([0, 50, 0, 50], [0, 1, -1], 1, 1.0, [51, -49]),
    ]),
    # ConvQuantizedTest_i8_to_float.basic, :4187-4197 (EXPECT_NEAR 0.001)
    "i8_to_float": dict(in_dtype="int8", out_dtype="float32", features=[
        ([125, 125, 0, 1], [2, 0, 1], 1, 1.0, [251.0, 252.0]),
        ([0, 50, 0, -50], [0, 8, 8], 2, 0.5, [201.0, -199.0]),
        ([0, 50, 0, -50], [0, 8, 8], 2, 1.0, [402.0, -398.0]),
        ([0, 5, 0, -5], [0, 8, 8], 0, 1.01, [40.4, -40.4]),
    ]),
}

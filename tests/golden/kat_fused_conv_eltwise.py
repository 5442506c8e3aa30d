"""Known-answer vectors of the reference's fused convolution+eltwise tests, kept
as literal data.  Source: tests/test_cases/fused_conv_eltwise_gpu_test.cpp
(clDNN tree), fixture FusedConvTest::do_test :159-269.

Feature tuple: (input[4], weights[3], bias, conv_input_quant, conv_calibration,
non_conv_input[2], eltw_output_calibration, pre_relu_output[2]); None stands for
the test's `ignore` (NaN) placeholder.  The primitive arguments that differ per
test are listed next to the features.  All tests: eltwise sum, eltw stride 1,
conv stride 1, no padding, no conv activation, eltwise ReLU.
"""

CASES = {
    # FusedConvTest_all_float.basic, :287-325
    "all_float": dict(in_dtype="float32", out_dtype="float32",
                      use_quant=True, use_conv_calib=True, use_eltw_calib=True,
                      conv_i_qf=1.0, non_conv_scale=1.0, features=[
        ([125.0, 125.0, 0.0, 1.0], [2.0, 0.0, 1.0], 1.0, 1.0, 1.0, [-10.0, -10.0], 1.0, [241.0, 242.0]),
        ([125.0, 125.0, 0.0, 1.0], [2.0, 0.0, 1.0], 0.0, 1.0, 1.0, [-10.0, -11.0], 2.0, [480.0, 480.0]),
    ]),
    # FusedConvTest_no_conv_calibration.basic, :330-377
    "no_conv_calibration": dict(in_dtype="float32", out_dtype="float32",
                                use_quant=True, use_conv_calib=False, use_eltw_calib=True,
                                conv_i_qf=1.0, non_conv_scale=1.0, features=[
        ([125.0, 125.0, 0.0, 1.0], [2.0, 0.0, 1.0], 1.0, 1.0, None, [-10.0, -10.0], 1.0, [241.0, 242.0]),
        ([125.0, 125.0, 0.0, 1.0], [2.0, 0.0, 1.0], 0.0, 1.0, None, [-10.0, -11.0], 2.0, [480.0, 480.0]),
    ]),
    # FusedConvTest_non_conv_scale_per_primitive.basic, :382-419
    "non_conv_scale_per_primitive": dict(in_dtype="int8", out_dtype="int8",
                                         use_quant=True, use_conv_calib=False, use_eltw_calib=True,
                                         conv_i_qf=1.0, non_conv_scale=2.0, features=[
        ([125, 125, 0, 1], [2, 0, 1], 1, 1.0, None, [-10, -10], 1.0, [231, 232]),
        ([125, 125, 0, 1], [2, 0, 1], 0, 1.0, None, [-10, -10], 1.0, [230, 231]),
        ([0, 50, 0, -50], [0, 4, 4], 1, 1.0, None, [-10, -10], 1.0, [181, -219]),
        ([0, 50, 0, -50], [0, 4, 4], 1, 1.0, None, [-5, -5], 1.0, [191, -209]),
        ([0, 50, 0, -50], [0, 8, 8], 2, 1.0, None, [10, 10], 0.5, [211, -189]),
    ]),
    # FusedConvTest_i8_to_u8_quantized.basic, :424-449
    "i8_to_u8_quantized": dict(in_dtype="int8", out_dtype="uint8",
                               use_quant=False, use_conv_calib=False, use_eltw_calib=True,
                               conv_i_qf=1.0, non_conv_scale=1.0, features=[
        ([125, 125, 0, 1], [2, 0, 1], 1, None, None, [-10, -10], 1.0, [241, 242]),
        ([125, 125, 0, 1], [2, 0, 1], 0, None, None, [-10, -11], 2.0, [480, 480]),
    ]),
    # FusedConvTest_i8_to_u8_no_eltw_calibration.basic, :455-499
    "i8_to_u8_no_eltw_calibration": dict(in_dtype="int8", out_dtype="uint8",
                                         use_quant=True, use_conv_calib=False, use_eltw_calib=False,
                                         conv_i_qf=1.0, non_conv_scale=1.0 / 3.0, features=[
        ([124, 124, 0, -4], [2, 0, 1], 4, 0.5, None, [-60, -60], None, [252 // 2 - 20, 248 // 2 - 20]),
        ([3, 3, 1, 1], [2, 0, 1], 0, 1.0 / 3.0, None, [1, 1], None, [2, 2]),
    ]),
}

"""Known-answer vectors of the reference's own int8 pooling and fully_connected tests, transcribed as data.

pooling: tests/test_cases/pooling_gpu_test.cpp:264-309 (basic_max_pooling_int8) and :311-358 (basic_avg_pooling_int8):
a 1x1x3x3 f32 input is reordered to int8, pooled with a 3x3 window, reordered back to f32.
fully_connected: tests/test_cases/fully_connected_gpu_test.cpp:239-297 (no_biases_int8): a 3-element f32 input reordered
to int8, 4x3 int8 weights, no bias, output reordered to f32.
"""

POOL_MAX_INT8 = dict(
    input_f32=[1.0, -2.5, 3.1, -4.0, 5.03, -6.99, 7.0, -8.0, 9.5],
    window=(3, 3), expected_f32=[9.0])

# expectation as the test computes it: the mean of the inputs truncated to char, truncated to char
POOL_AVG_INT8 = dict(
    input_f32=[2.0, -2.5, 5.1, -4.0, 8.03, -6.99, 17.0, -8.0, 19.5],
    window=(3, 3))

FC_NO_BIAS_INT8 = dict(
    input_f32=[8.4, 2.3, -4.99],
    weights_i8=[[2, 1, 0], [-3, -2, 1], [0, -2, -4], [-5, 10, 8]],
    expected_f32=[18.0, -32.0, 12.0, -52.0])

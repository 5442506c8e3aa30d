"""Known-answer data of the reference's own softmax tests (tests/test_cases/softmax_gpu_test.cpp), transcribed as data.

VALUES_BATCH_WISE (:137-164): ten classes, two identical batches (the reference stores them x-major, batch-minor; here
one batch is listed) and the expected probabilities.
SCOPES (:181-447): one 2x3x2x2 bfyx input and, per normalisation scope, the largest probability of every normalised set
in the order the reference's checks walk them; every set must also sum to 1.
"""

VALUES_BATCH_WISE = {
    "input": [2.0, 2.0, 2.0, 3.0, 5.0, 4.0, 3.0, 2.0, 2.0, 2.0],
    "expected": [0.02569957, 0.02569957, 0.02569957, 0.069858674, 0.516189665, 0.189895565, 0.069858674, 0.02569957, 0.02569957, 0.02569957],
}

SCOPES_INPUT_BFYX = [  # shape (2, 3, 2, 2)
    0.1, -0.1, 0.9, 1.5,
    0.2, 0.2, -10.0, 5.2,
    0.2, 0.2, -10.0, 5.2,
    3.0, 0.5, 7.0, 12.0,
    4.0, 0.5, 8.0, 8.2,
    0.2, 0.2, -10.0, 5.2,
]

# normalize_fyx (:181-249): one set per batch
EXPECTED_MAX_FYX = [0.481618381, 0.953259517]
# normalize_y (:251-354): sets in (b, f, x) order
EXPECTED_MAX_Y = [0.689974481, 0.832018385, 0.999962831, 0.993307149, 0.999962831, 0.993307149,
                  0.98201379, 0.99998987, 0.98201379, 0.999547378, 0.999962831, 0.993307149]
# normalize_f (:356-447): sets in (b, y, x) order
EXPECTED_MAX_F = [0.344253346, 0.364854551, 0.999963085, 0.493894592, 0.719294981, 0.364854551, 0.73105857, 0.977054322]

"""CPU: the reference's functional gate for the quantized path (quantized_MNIST_test, tests/nn_tests.cpp:536-974:
uint8 accuracy / float32 accuracy > 0.95) replayed through the oracle on seeded synthetic digit images."""
import numpy as np

from helpers import oracle_digit_replay, synthetic_digits, train_float_digit_net


def test_uint8_network_keeps_the_float_accuracy(oracle):
    xtr, ytr = synthetic_digits(1, 8000)
    xte, yte = synthetic_digits(2, 600)
    ranges = [[np.inf, -np.inf] for _ in range(4)]

    def observe(taps):
        for r, t in zip(ranges, taps):
            r[0], r[1] = min(r[0], float(t.min())), max(r[1], float(t.max()))

    weights, predict = train_float_digit_net(xtr, ytr, observe=observe)
    fp32_score = 100.0 * (predict(xte) == yte).mean()
    assert fp32_score > 80, "the float network did not learn the synthetic classes"
    _, logits = oracle_digit_replay(oracle, xte, weights, ranges)
    uint8_score = 100.0 * (logits.argmax(1) == yte).mean()
    assert uint8_score / fp32_score > 0.95        # the reference's pass criterion (tests/nn_tests.cpp:968)

"""GPU: the reference's functional gate for the quantized path (quantized_MNIST_test, tests/nn_tests.cpp:536-974)
replayed on seeded synthetic digit images: float32 training with range observers, quantisation set-up through the
calibration helper, inference through Conv2d_q -> FullyConnected_q -> FullyConnected_q on the device.  Every uint8
byte must equal the oracle's, and the uint8 network must keep more than 95 % of the float32 accuracy."""
import numpy as np
import pytest

from helpers import oracle_digit_replay, synthetic_digits, train_float_digit_net

pytestmark = pytest.mark.gpu


def test_quantized_digit_network_on_the_device(cuda, oracle):
    import ltq
    xtr, ytr = synthetic_digits(1, 8000)
    xte, yte = synthetic_digits(2, 1000)
    observers = [ltq.MinMaxObserver() for _ in range(4)]          # input, conv1, fc1, fc2 (nn_tests.cpp:550)

    def observe(taps):
        for o, t in zip(observers, taps):
            o.update(t.cuda())

    weights, predict = train_float_digit_net(xtr, ytr, observe=observe)
    fp32_score = 100.0 * (predict(xte) == yte).mean()
    assert fp32_score > 80, "the float network did not learn the synthetic classes"
    qps = [o.qparams() for o in observers]

    conv1 = ltq.Conv2d_q(1, 10, False, 5, 5)
    fc1 = ltq.FullyConnected_q(5760, 50)
    fc2 = ltq.FullyConnected_q(50, 10)
    mods = (conv1, fc1, fc2)
    for i, m in enumerate(mods):
        m.init()
        ltq.quantize_module(m, cuda.from_numpy(weights[i]).cuda(), None, qps[i], qps[i + 1])
        m.to("cuda", 0)

    def qnet(x_u8):                                               # QNet::forward, nn_tests.cpp:630-640
        out = conv1.forward(x_u8)
        out = out.reshape(out.shape[0], 1, 1, 5760)
        return fc2.forward(fc1.forward(out))

    ranges = [(o.min, o.max) for o in observers]
    (_, _, y3_o), logits_o = oracle_digit_replay(oracle, xte, weights, ranges)

    # the whole test set as one batch
    q_input = ltq.Quantize(cuda.from_numpy(xte).cuda(), qps[0])
    q_output = qnet(q_input)
    np.testing.assert_array_equal(q_output.cpu().numpy().reshape(len(xte), 10), y3_o)
    logits = ltq.Dequantize(q_output, qps[3]).cpu().numpy().reshape(len(xte), 10)
    np.testing.assert_array_equal(logits, logits_o)
    uint8_score = 100.0 * (logits.argmax(1) == yte).mean()
    assert uint8_score / fp32_score > 0.95                        # the reference's pass criterion (nn_tests.cpp:968)

    # and image by image, as the reference's loop runs it (nn_tests.cpp:935-963)
    for i in range(48):
        one = qnet(ltq.Quantize(cuda.from_numpy(xte[i:i + 1]).cuda(), qps[0]))
        np.testing.assert_array_equal(one.cpu().numpy().reshape(10), y3_o[i], err_msg=f"image {i}")
    fc1._handle.check()                                           # no bounded wait ran out on the device

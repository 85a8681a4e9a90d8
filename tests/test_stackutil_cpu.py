"""Host-side helpers of the stack tests and the bench: the two forms of the network input hold the
same values, and the first-layer case of a plain-image stack names the nchw format."""
import numpy as np

import refutil as R
import stackutil as S


def test_plain_and_blocked_network_input_hold_the_same_values():
    for int8 in (False, True):
        plain = S.vgg_input(3, 2, int8, plain=True)
        blocked = S.vgg_input(3, 2, int8)
        assert plain.shape == (2, 3, 224, 224) and blocked.shape == (2, 1, 224, 224, 16)
        assert plain.dtype == blocked.dtype == (np.uint8 if int8 else np.float32)
        assert np.array_equal(R.to_nChw16c(plain), blocked)
        assert not blocked[..., 3:].any()            # the thirteen padding channels are zero
        assert plain.nbytes * 5 < blocked.nbytes


def test_first_layer_case_of_a_plain_image_stack():
    ic, oc, hw, _ = S.vgg_layers()[0]
    c = S.vgg_layer_case(0, ic, oc, hw, 2, False, plain_image=True)
    assert c.ifmt == "nchw" and c.ofmt == "" and c.ic == 3 and c.oc == 64
    assert S.vgg_layer_case(0, ic, oc, hw, 2, False).ifmt == ""
    ic1, oc1, hw1, _ = S.vgg_layers()[1]
    assert S.vgg_layer_case(1, ic1, oc1, hw1, 2, False, plain_image=True).ifmt == ""      # only the first layer

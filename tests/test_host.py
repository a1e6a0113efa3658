"""Host-side mirror of the reference's Python surface: enums, signatures, module parameters, errors.
CPU only."""
import inspect

import pytest
import torch

import morphocore_b200 as M
import morphocore_b200.functional as F
import morphocore_b200.nn as Mnn
import workloads as WL
from morphocore_b200.functional.merge_enum import MorphoMerge, MorphoPadding, str_to_merge, str_to_padding


def test_enum_integers_match_the_operator_schema():
    assert [str_to_merge(m).value for m in ("max", "min", "sum", "mean", "identity")] == [0, 1, 2, 3, 5]
    assert [str_to_padding(p).value for p in ("zero", "geodesic", "constant", "replicate")] == [0, 1, 2, 3]
    assert MorphoMerge.SMOOTH == 4 and MorphoPadding.REPLICATE == 3


def test_reference_package_name_resolves_to_this_implementation():
    """`import morphocore.functional` / `import morphocore.nn` (the reference's names, used by its own tests and by its
    users) serve the B200 functions and modules."""
    import morphocore
    import morphocore.functional as RF
    import morphocore.nn as RN
    from morphocore.nn import Closing, Opening
    assert RF.dilation is F.dilation and RF.erosion is F.erosion and RF.smorph is F.smorph and RF.sigma_layer is F.sigma_layer
    assert RN.Dilation is Mnn.Dilation and RN.SMorph is Mnn.SMorph and Opening is Mnn.Opening and Closing is Mnn.Closing
    assert morphocore.__version__ == M.__version__


def test_unknown_modes_raise_value_error():
    with pytest.raises(ValueError, match="Unknown merge mode"):
        str_to_merge("average")
    with pytest.raises(ValueError, match="Unknown padding mode"):
        str_to_padding("reflect")
    with pytest.raises(ValueError, match="Unknown padding mode"):
        F.dilation(torch.zeros(1, 1, 4, 4), torch.zeros(1, 1, 3, 3), padding_mode="bogus")


def test_functional_signatures_are_the_reference_ones():
    names = list(inspect.signature(F.dilation).parameters)
    assert names == ["x", "w", "channel_merge_mode", "padding_mode", "save_indices", "weight_dropout", "training", "padding_value",
                     "noise_scale"]
    assert list(inspect.signature(F.erosion).parameters) == names
    assert list(inspect.signature(F.smorph).parameters) == ["x", "w", "alpha", "beta", "channel_merge_mode"]
    sig = inspect.signature(F.dilation)
    assert sig.parameters["channel_merge_mode"].default == "sum" and sig.parameters["padding_mode"].default == "replicate"
    assert sig.parameters["save_indices"].default is True


def test_operator_schemas():
    ops = torch.ops.morphocore
    assert str(ops.dilation.default._schema) == (
        "morphocore::dilation(Tensor input, Tensor weight, int merge, int padding, float padding_value=0., "
        "bool save_indices=True, float noise_scale=0.) -> Tensor")
    assert str(ops.smorph.default._schema) == "morphocore::smorph(Tensor input, Tensor weight, Tensor alpha, int merge) -> Tensor"
    assert "smorph_scm" in dir(ops) or ops.smorph_scm is not None


def test_module_parameters():
    d = Mnn.Dilation(3, 16, 5)
    assert d.weight.shape == (16, 3, 5, 5) and torch.count_nonzero(d.weight) == 0
    assert d.channel_merge_mode == "sum" and d.padding_mode == "replicate" and d.save_indices is True
    e = Mnn.Erosion(4, 4, (3, 5), channel_merge_mode="identity", dtype=torch.float64)
    assert e.weight.shape == (4, 1, 3, 5) and e.weight.dtype == torch.float64
    with pytest.raises(ValueError, match="identity"):
        Mnn.Dilation(3, 4, 3, channel_merge_mode="identity")
    s = Mnn.SMorph(3, 8, 3, init_alpha=2.0)
    assert s.alpha.shape == (8, 3) and float(s.alpha[0, 0]) == 2.0 and s.beta is None
    assert set(s.state_dict()) == {"weight", "alpha"}
    si = Mnn.SMorph(5, 5, 3, channel_merge_mode="identity")
    assert si.alpha.shape == (5, 1) and si.weight.shape == (5, 1, 3, 3)
    sb = Mnn.SMorph(3, 8, 3, init_beta=1.0)
    assert sb.beta.shape == (8, 3)


def test_cpu_tensors_are_rejected_loudly():
    x, w = torch.zeros(1, 1, 4, 4), torch.zeros(1, 1, 3, 3)
    for call in (lambda: F.dilation(x, w), lambda: F.erosion(x, w), lambda: F.smorph(x, w, torch.zeros(1, 1))):
        with pytest.raises(RuntimeError, match="no CPU path"):
            call()
    with pytest.raises(RuntimeError, match="noise_scale"):
        F.dilation(x, w, noise_scale=-1.0, training=True)
    with pytest.raises(RuntimeError, match="no CPU path"):
        F.smorph(x, w, torch.zeros(1, 1), beta=torch.zeros(1))


def test_workload_tap_counts():
    assert WL.cfg1()["n_taps"] == 56_623_104
    assert WL.taps(32, 32, 16, 256, 256, 5, 5) == 26_843_545_600
    assert WL.taps(16, 32, 32, 128, 128, 7, 7) == 13_153_337_344
    assert WL.taps(8, 64, 64, 512, 512, 11, 11, identity=True) == 16_240_345_088
    assert WL.cfg5_taps(256) == 2_284_570_279_936
    assert M.__version__

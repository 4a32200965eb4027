"""The sampler and its processor kernels on the GPU, against the torch statements of the kernels."""

import pytest
import torch

import sampling_cases as sc
from emulated_ops import TorchOps

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


@pytest.mark.parametrize("case", [sc.case_greedy_and_equivalents, sc.case_seeded_draws,
                                  sc.case_filters_restrict_the_support, sc.case_bias_and_penalties],
                         ids=lambda f: f.__name__[5:])
def test_sampler(ops, case):
    case(ops, "cuda")


@pytest.mark.parametrize("V", [301, 4099, 151936])
def test_filter_kernel_matches_its_statement(ops, V):
    g = torch.Generator().manual_seed(V)
    x = (torch.randn(6, V, generator=g) * 3).cuda()
    temp = torch.tensor([1.0, 0.7, 1.3, 0.9, 2.0, 1.0]).cuda()
    min_p = torch.tensor([0.0, 0.1, 0.0, 0.0, 0.05, 0.0]).cuda()
    top_k = torch.tensor([0, 0, 50, 0, 7, 1], dtype=torch.int32).cuda()
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.8, 0.6, 1.0]).cuda()
    got = ops.filter_rows(x.clone(), temp, min_p, top_k, top_p)
    want = TorchOps().filter_rows(x.clone(), temp, min_p, top_k, top_p)
    kept_got, kept_want = got > -1e30, want > -1e30
    # the kept sets agree except for tokens that sit within rounding of a cut-off
    assert int((kept_got != kept_want).sum()) <= 2
    both = kept_got & kept_want
    assert float((got[both] - want[both]).abs().max()) < 1e-5
    assert torch.equal(got[0], x[0]) and int(kept_got[5].sum()) == 1 and int(kept_got[2].sum()) == 50


def test_bias_penalty_kernel_matches_its_statement(ops):
    V = 4099
    x = torch.randn(V, generator=torch.Generator().manual_seed(1)).cuda()
    seen = torch.randint(0, V, (500,), generator=torch.Generator().manual_seed(2)).tolist() + [V + 3, -1]
    kw = dict(logit_bias={5: 2.5, 4000: -7.0}, seen_ids=seen, repetition_penalty=1.3, presence_penalty=0.4,
              frequency_penalty=0.1)
    got = ops.bias_penalty_row(x.clone(), **kw)
    want = TorchOps().bias_penalty_row(x.clone(), **kw)
    assert float((got - want).abs().max()) < 1e-6


def test_bias_and_penalties_for_several_rows_in_one_launch(ops):
    """Rows with a bias only, penalties only, both, and nothing that bites: one launch, each row as
    the one-row statement gives it; rows that are not named stay as they were."""
    g = torch.Generator().manual_seed(11)
    V = 1531
    x = (torch.randn((6, V), generator=g) * 3).cuda()
    rows = [4, 0, 2, 5]
    kw = dict(logit_bias=[{3: 2.5, 1500: -4.0}, None, {7: 1.0}, None],
              seen_ids=[[1, 2, 3], [5, 5, 5, 9, 1000], torch.randint(0, V, (300,), generator=g).tolist(), [4, 4]],
              repetition_penalty=[1.0, 1.3, 0.8, 1.0], presence_penalty=[0.0, 0.5, 0.0, 0.0],
              frequency_penalty=[0.0, 0.0, 0.25, 0.0])
    got = ops.bias_penalty_rows(x.clone(), rows, **kw)
    want = TorchOps().bias_penalty_rows(x.clone(), rows, **kw)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-6)
    assert torch.equal(got[[1, 3]], x[[1, 3]])
    assert not torch.equal(got[0], x[0]) and torch.equal(got[5], x[5])  # row 5: penalties that change nothing

"""The host side of a step: token ids from lists, arrays and tensors become one array; anything
that is not an integer is refused before a kernel sees it."""
import numpy as np
import pytest
import torch

from llm_infer_engine_b200.engine.engine import EngineError, _flatten_tokens


def _flat(tokens):
    lens = [len(t) for t in tokens]
    return _flatten_tokens(tokens, lens)


def test_lists_arrays_and_tensors_give_the_same_ids():
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 1000, size=n).tolist() for n in (300, 1, 129)]
    want = np.concatenate([np.asarray(s) for s in seqs])
    assert np.array_equal(_flat(seqs), want)
    assert np.array_equal(_flat([np.asarray(s, dtype=np.int32) for s in seqs]), want)
    assert np.array_equal(_flat([torch.tensor(s) for s in seqs]), want)
    assert np.array_equal(_flat([seqs[0], np.asarray(seqs[1]), torch.tensor(seqs[2])]), want)


def test_many_short_sequences():
    seqs = [[i] for i in range(64)] + [[7, 8, 9]]
    assert _flat(seqs).tolist() == list(range(64)) + [7, 8, 9]


def test_negative_and_large_ids_survive_for_the_range_check():
    assert _flat([[-1, 2 ** 40] + [0] * 200]).tolist()[:2] == [-1, 2 ** 40]


@pytest.mark.parametrize("bad", [[[1.5] * 200], [["a"] * 200], [np.zeros(200, dtype=np.float32)], [[2 ** 70] * 200],
                                 [[1.5]]])
def test_non_integers_are_refused(bad):
    with pytest.raises(EngineError):
        _flat(bad)

"""Arrow column <-> tensor conversion (host-side I/O, no GPU needed) and the saved-index round trip."""
import numpy as np
import pyarrow as pa
import pytest
import torch


def test_list_column_fills_a_tensor_batch_by_batch():
    from vectorlink_gpu.datafusion import dataframe_to_tensor, tensor_to_arrow
    rng = np.random.default_rng(0)
    data = rng.standard_normal((10, 6)).astype(np.float32)
    fixed = tensor_to_arrow(torch.from_numpy(data))
    assert fixed.type.list_size == 6
    chunked = pa.chunked_array([fixed.slice(0, 4), fixed.slice(4, 6)])       # sliced chunks carry offsets
    out = torch.empty((10, 6), dtype=torch.float32)
    dataframe_to_tensor(chunked, out)
    assert np.array_equal(out.numpy(), data)
    plain = pa.array([list(r) for r in data.tolist()], type=pa.list_(pa.float32()))   # variable-size list type
    out2 = torch.empty((10, 6), dtype=torch.float32)
    dataframe_to_tensor(pa.table({"embedding": plain}), out2)
    assert np.array_equal(out2.numpy(), data)
    ints = torch.arange(12, dtype=torch.int32).reshape(4, 3)
    back = torch.empty((4, 3), dtype=torch.int32)
    dataframe_to_tensor(tensor_to_arrow(ints), back)
    assert torch.equal(back, ints)
    with pytest.raises(ValueError):
        dataframe_to_tensor(tensor_to_arrow(ints), torch.empty((5, 3), dtype=torch.int32))
    with pytest.raises(ValueError):
        dataframe_to_tensor(tensor_to_arrow(ints), torch.empty((4, 3), dtype=torch.float32))


@pytest.mark.gpu
def test_saved_index_round_trip(c1, built_lib):
    from vectorlink_gpu import ANN
    from conftest import cfg_of
    _, kw = cfg_of(c1)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ann = ANN(t(c1["vectors"]), beams=t(c1["beams"]), distances=t(c1["distances"]), **kw)
    table = ann.to_arrow()
    shuffled = table.take(pa.array(np.random.default_rng(1).permutation(table.num_rows)))
    kw2 = {k: v for k, v in kw.items() if k != "beam_size"}
    again = ANN.load_from_dataframe(shuffled, **kw2)
    assert torch.equal(again.vectors, ann.vectors) and torch.equal(again.beams, ann.beams)
    assert torch.equal(again.distances, ann.distances)
    sq = again.search(t(c1["queries"]))
    assert np.array_equal(sq.indices.cpu().numpy(), c1["search_tree_ids"])

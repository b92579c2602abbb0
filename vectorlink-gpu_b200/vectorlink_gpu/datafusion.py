"""Arrow <-> tensor I/O of the reference (vectorlink_gpu/datafusion.py:27-56) on pyarrow.

The reference streams DataFusion record batches into a CUDA tensor through Numba's
`copy_to_device`.  Here the same column layout is read from anything that yields Arrow
record batches - a `pyarrow.Table` / `RecordBatchReader`, or a DataFusion `DataFrame` when
that package is installed (it is optional) - by viewing each batch's value buffer without a
copy and handing it to `Tensor.copy_` (pinned staging for CUDA targets).
Columns: `vector_id`, `embedding` (list<float32>[dim]), `beams` (list<int32>[D]) and
optionally `distances` (list<float32>[D]); rows are taken in the order given (sort by
`vector_id` first, as ANN.load_from_dataframe does).
"""
from __future__ import annotations

import ctypes
from typing import Iterable

import numpy as np
import pyarrow as pa
import torch
from torch import Tensor


def dtype_to_ctype(dtype):
    """datafusion.py:27-33."""
    if dtype == torch.float32:
        return ctypes.c_float
    elif dtype == torch.int32:
        return ctypes.c_int32
    else:
        raise ValueError(f"i don't know what a {dtype} is")


def _np_dtype(dtype):
    return {torch.float32: np.float32, torch.int32: np.int32}[dtype]


def _batches(source, column: int = 0) -> Iterable[pa.Array]:
    """The chunks of one column of `source` as Arrow arrays."""
    if hasattr(source, "execute_stream"):                 # DataFusion DataFrame (datafusion.py:39)
        for batch in source.execute_stream():
            yield batch.to_pyarrow().column(column)
    elif isinstance(source, pa.Table):
        yield from source.column(column).chunks
    elif isinstance(source, pa.ChunkedArray):
        yield from source.chunks
    elif isinstance(source, pa.Array):
        yield source
    else:                                                 # RecordBatchReader / iterable of batches
        for batch in source:
            yield batch.column(column)


def _list_values(arr: pa.Array, width: int, np_dtype) -> np.ndarray:
    """[len(arr), width] view of a (fixed-size or plain) list array's values, no copy."""
    flat = arr.flatten()
    values = flat.to_numpy(zero_copy_only=True)
    if values.dtype != np_dtype:
        raise ValueError(f"column holds {values.dtype}, the tensor wants {np.dtype(np_dtype)}")
    if values.size != len(arr) * width:
        raise ValueError(f"{values.size} values for {len(arr)} rows of width {width}")
    return values.reshape(len(arr), width)


def dataframe_to_tensor(df, tensor: Tensor, column: int = 0):
    """datafusion.py:36-52: fill `tensor` [rows, width] from the (sorted) list column, batch by batch."""
    offset = 0
    width = tensor.size(1)
    np_dtype = _np_dtype(tensor.dtype)
    for arr in _batches(df, column):
        if len(arr) == 0:
            continue
        block = torch.from_numpy(_list_values(arr, width, np_dtype))
        if tensor.is_cuda:
            block = block.pin_memory()
        tensor[offset: offset + len(arr)].copy_(block, non_blocking=tensor.is_cuda)
        offset += len(arr)
    if tensor.is_cuda:
        torch.cuda.current_stream(tensor.device).synchronize()
    if offset != tensor.size(0):
        raise ValueError(f"column holds {offset} rows, the tensor {tensor.size(0)}")


def tensor_to_arrow(tensor: Tensor) -> pa.Array:
    """datafusion.py:55-56: a [rows, width] tensor as a fixed-size-list array."""
    host = tensor.detach().cpu().contiguous().numpy()
    return pa.FixedSizeListArray.from_arrays(pa.array(host.reshape(-1)), host.shape[1])

"""Reading MATLAB .mat files into numpy arrays, same call as the reference's dataset/data_accessor.py:32-38.

Files up to format v7.2 go through scipy.io.loadmat.  Format v7.3 files are HDF5 containers: they need h5py, which
is optional here; arrays read that way come out with reversed axes (MATLAB is column-major) and are transposed back.
"""
from typing import List, Sequence

import numpy as np


def read_matfile_old(filepath: str, key_list: Sequence[str], dtype_list: Sequence) -> List[np.ndarray]:
    from scipy.io import loadmat
    data = loadmat(filepath, variable_names=list(key_list))
    return [np.ascontiguousarray(data[key]).astype(dtype) for key, dtype in zip(key_list, dtype_list)]


def read_matfile_v73(filepath: str, key_list: Sequence[str], dtype_list: Sequence) -> List[np.ndarray]:
    try:
        import h5py
    except ImportError as ex:
        raise ImportError(f'{filepath} is a MATLAB v7.3 (HDF5) file; reading it needs the h5py package') from ex
    out = []
    with h5py.File(filepath, 'r') as data:
        for key, dtype in zip(key_list, dtype_list):
            val = data[key][()]
            out.append(np.ascontiguousarray(np.transpose(val)).astype(dtype))    # reverse every axis
    return out


def read_matfile(filepath: str, key_list: Sequence[str], dtype_list: Sequence) -> List[np.ndarray]:
    """Values of `key_list` cast to `dtype_list`; tries the old formats first, then v7.3."""
    try:
        return read_matfile_old(filepath, key_list, dtype_list)
    except NotImplementedError:          # scipy's signal for "this is an HDF5 (v7.3) file"
        return read_matfile_v73(filepath, key_list, dtype_list)

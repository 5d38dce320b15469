"""b2lstm: Python harness over libb2lstm.so, the B200 implementation of the CURRENNT peephole
LSTM / BLSTM training path.  The library is the product; this package only loads it (ctypes),
generates the synthetic workloads and launches processes.  There is no CPU fallback: importing
works without a GPU (symbols can be inspected), every compute call needs one.
"""
from .lib import (B2Error, LstmLayer, Net, lib, library_path, lstm_num_weights, matrix_multiply, matrix_multiply_noalloc,
                  dp_unique_id, DataSet, data_reseed, train_epoch, train_epoch_batch, write_nc, Optimizer)
from . import workloads

__all__ = ["B2Error", "LstmLayer", "Net", "lib", "library_path", "lstm_num_weights", "matrix_multiply", "matrix_multiply_noalloc",
           "dp_unique_id", "DataSet", "data_reseed", "train_epoch", "train_epoch_batch", "write_nc", "Optimizer", "workloads"]

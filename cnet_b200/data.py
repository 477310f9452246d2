"""MnistDataReader of the reference (data/data.h:82-165) over the host facade: the idx3 / idx1 files read the way
the reference reads them, handed out as split planes for `Net.upload` / `prefetch`."""
import ctypes as C

import numpy as np

from . import lib as _lib


class MnistDataReader:
    def __init__(self, image_file, label_file, count):
        self.lib = _lib.load()
        self.h = C.c_void_p(self.lib.cnh_mnist_open(str(image_file).encode(), str(label_file).encode(), int(count)))
        if not self.h:
            raise _lib.CnetError("cannot read %d samples from %s / %s" % (count, image_file, label_file))

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.cnh_mnist_close(self.h)
            self.h = None

    def size(self):
        return self.lib.cnh_mnist_size(self.h)

    def shuffle(self, seed=0):
        self.lib.cnh_mnist_shuffle(self.h, seed)

    def has_next_batch(self, batch):
        return bool(self.lib.cnh_mnist_has_next(self.h, batch))

    def next_batch(self, batch):
        """((re, im) planes [batch, 784] float32, labels [batch] int32); wraps around at the end."""
        re, im = np.empty((batch, 784), np.float32), np.empty((batch, 784), np.float32)
        labels = np.empty(batch, np.int32)
        if self.lib.cnh_mnist_next_batch(self.h, batch, re.ctypes.data, im.ctypes.data, labels.ctypes.data) != 0:
            raise _lib.CnetError("next_batch failed")
        return (re, im), labels

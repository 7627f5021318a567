"""Element types and tensor types of the operator language.

The integer codes of :class:`DType` are the wire values of the reference's ``DType`` enum
(opveclib/language.proto:16-37), because they cross the C-ABI in ``OvlTensor.dtype`` exactly as they cross
the reference's ``_TensorParam.dtype`` (opveclib/operator.py:128-131).  The C spellings are the ones the
reference emits (opveclib/expression.py:50-61); ``int64`` is ``long long`` there (opveclib/dynamiclibop.h:18).
"""
import numpy as np

_TABLE = [
    # code, name, numpy type, C type, bytes, is_float, is_signed
    (1, 'float16', np.float16, None, 2, True, True),
    (2, 'float32', np.float32, 'float', 4, True, True),
    (3, 'float64', np.float64, 'double', 8, True, True),
    (4, 'int8', np.int8, 'int8_t', 1, False, True),
    (5, 'int16', np.int16, 'int16_t', 2, False, True),
    (6, 'int32', np.int32, 'int32_t', 4, False, True),
    (7, 'int64', np.int64, 'long long', 8, False, True),
    (8, 'uint8', np.uint8, 'uint8_t', 1, False, False),
    (9, 'uint16', np.uint16, 'uint16_t', 2, False, False),
    (10, 'uint32', np.uint32, 'uint32_t', 4, False, False),
    (11, 'uint64', np.uint64, 'uint64_t', 8, False, False),
]
_BY_CODE = {row[0]: row for row in _TABLE}
_BY_NAME = {row[1]: row for row in _TABLE}


class DType(object):
    """A low level element type.  Construct from another DType, a numpy type/dtype, a torch dtype, the
    type's name or its integer wire code."""
    __slots__ = ('code',)

    def __init__(self, spec):
        if isinstance(spec, DType):
            self.code = spec.code
            return
        if isinstance(spec, bool):
            raise TypeError('dtype ' + str(spec) + ' is not valid.')
        if isinstance(spec, (int, np.integer)):
            if int(spec) not in _BY_CODE:
                raise ValueError('dtype ' + str(spec) + ' is not valid.')
            self.code = int(spec)
            return
        if isinstance(spec, str) and spec in _BY_NAME:
            self.code = _BY_NAME[spec][0]
            return
        name = None
        try:
            name = np.dtype(spec).name
        except TypeError:
            # torch dtypes print as 'torch.float32'
            text = str(spec)
            if text.startswith('torch.'):
                name = text[len('torch.'):]
        if name not in _BY_NAME:
            raise TypeError('dtype ' + str(spec) + ' is not valid.')
        self.code = _BY_NAME[name][0]

    def __eq__(self, other):
        return isinstance(other, DType) and other.code == self.code

    def __ne__(self, other):
        return not self == other

    def __hash__(self):
        return hash(('ovl.DType', self.code))

    def __str__(self):
        return self.name.upper()

    __repr__ = __str__

    @property
    def name(self):
        return _BY_CODE[self.code][1]

    @property
    def itemsize(self):
        return _BY_CODE[self.code][4]

    @property
    def is_float(self):
        return _BY_CODE[self.code][5]

    @property
    def is_signed(self):
        return _BY_CODE[self.code][6]

    @property
    def is_unsigned(self):
        return not _BY_CODE[self.code][6]

    def as_numpy(self):
        return _BY_CODE[self.code][2]

    def as_cstr(self):
        c = _BY_CODE[self.code][3]
        if c is None:
            raise TypeError(self.name + ' has no C representation')
        return c

    def as_torch(self):
        import torch
        return getattr(torch, self.name)

    def as_proto(self):
        return self.code


float16 = DType(1)
float32 = DType(2)
float64 = DType(3)
int8 = DType(4)
int16 = DType(5)
int32 = DType(6)
int64 = DType(7)
uint8 = DType(8)
uint16 = DType(9)
uint32 = DType(10)
uint64 = DType(11)

supported_types = [float16, float32, float64, int8, int16, int32, int64, uint8, uint16, uint32, uint64]


def _is_int(x):
    return isinstance(x, (int, np.integer)) and not isinstance(x, (bool, np.bool_))


class TensorType(object):
    """Shape plus element type; every dimension is a positive compile-time integer
    (opveclib/expression.py:146-238)."""

    def __init__(self, shape, dtype):
        self.dtype = DType(dtype)
        if _is_int(shape):
            self.shape = [int(shape)]
        else:
            self.shape = []
            for elem in shape:
                if elem is None:
                    raise TypeError('All dimensions must be defined.')
                if not _is_int(elem):
                    raise TypeError('Shape must be an iterable of ints.')
                self.shape.append(int(elem))
        for elem in self.shape:
            if elem <= 0:
                raise ValueError('All tensor dimensions must be positive, but got: ' + str(self.shape))
        self.size = 1
        for elem in self.shape:
            self.size *= elem
        self.rank = len(self.shape)

    def __eq__(self, other):
        return isinstance(other, TensorType) and other.shape == self.shape and other.dtype == self.dtype

    def __ne__(self, other):
        return not self == other

    def __hash__(self):
        return hash((tuple(self.shape), self.dtype.code))

    def __str__(self):
        return 'TensorType(' + str(self.shape) + ', ' + self.dtype.name + ')'

    __repr__ = __str__

    @property
    def tensor_type(self):
        return self

    @staticmethod
    def like(other):
        """TensorType of anything that has a shape and a dtype: numpy arrays, torch tensors, tensor
        expressions, operator outputs, TensorTypes."""
        if isinstance(other, TensorType):
            return TensorType(other.shape, other.dtype)
        try:
            shape = other.shape
        except AttributeError:
            shape = other.get_shape().as_list()
        return TensorType(list(shape), other.dtype)

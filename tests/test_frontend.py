"""Host-side behaviour of the operator language and the operator graph (no GPU, no compilation).

Mirrors the reference's unit tests of the same layer: opveclib/test/test_expressions.py (type validation, node
construction rules, python-truthiness guard) and opveclib/test/test_operator.py (graph structure, output
ordering, wrong returns, the re-assignment guard).
"""
import numpy as np
import pytest

import opveclib_b200 as ovl
from opveclib_b200 import expr as E
from opveclib_b200.dtypes import DType, TensorType, float16, float32, float64, int64, uint8, uint32, uint64
from opveclib_b200.kernel import iter_nodes
from opveclib_b200.opgraph import build_op_dag


def test_dtype_validation():
    for bad in ('string', 1.0, np.ndarray):
        with pytest.raises(TypeError):
            DType(bad)
    with pytest.raises(ValueError):
        DType(100000)
    assert float16 == DType(np.float16) and float32 == DType(np.float32) and float64 == DType(np.float64)
    assert uint8 == DType(np.zeros(10, dtype=np.uint8).dtype)
    assert uint64.as_numpy() == np.uint64 and float32.as_cstr() == 'float' and int64.as_cstr() == 'long long'
    assert DType(2) == float32 and DType(float32) == float32 and float32 != float64
    import torch
    assert DType(torch.float32) == float32 and DType(torch.int64) == int64


def test_tensor_type_validation():
    for bad in ('string', (1, 2, 3.3), np.array([1.0, 2.0, 3.0])):
        with pytest.raises(TypeError):
            TensorType(bad, float32)
    with pytest.raises(ValueError):
        TensorType([0, 5], float32)
    assert TensorType((1, 2, 3), float32) == TensorType([1, 2, 3], np.float32)
    assert TensorType(5, float32) == TensorType([5], float32) != TensorType([5], float16)
    assert TensorType((5, 10, 100), float32).size == 5000
    assert TensorType.like(np.zeros((10, 10), dtype=np.float64)) == TensorType([10, 10], float64)


def test_expressions_need_a_trace():
    with pytest.raises(RuntimeError):
        E.ConstScalar(1)


def test_io_nodes_and_access_rules():
    with E.tracing():
        t = TensorType([5, 5], uint64)
        in0 = E.InputTensor(t, 0)
        with pytest.raises(ValueError):
            E.InputTensor(t, -1)
        with pytest.raises(ValueError):
            E.InputTensor(t, 2 ** 32)
        with pytest.raises(TypeError):
            E.InputTensor('string', 1)
        with pytest.raises(ValueError):
            E.InputTensor(t, 5)          # out of order
        out0 = E.OutputTensor(t, 0)
        out0[0, 0] = 0
        with pytest.raises(TypeError):
            out0[0, 0]                   # outputs cannot be read
        with pytest.raises(TypeError):
            in0[0, 0] = 1                # inputs cannot be written
        with pytest.raises(IndexError):
            in0[5, 0]
        with pytest.raises(IndexError):
            in0[0]                       # rank mismatch
        E.position_in([5, 5])
        with pytest.raises(ValueError):
            E.position_in([5, 5])        # only one workgroup per operator


def test_typing_rules_of_binary_math():
    with E.tracing():
        x = E.input([4], float32)
        pos = E.position_in(4)
        a = x[pos]
        s = a + 1                        # python int -> int64 const -> cast to float32
        assert s.dtype == float32 and s.args[1].kind == 'cast' and s.args[1].args[0].dtype == int64
        f = 2.5 * a
        assert f.dtype == float32 and f.args[0].args[0].dtype == float64
        c = a < s
        assert c.dtype == float32        # comparisons keep the operand dtype
        with pytest.raises(TypeError):
            E.BinaryMath('add', 1, 2)
        with pytest.raises(TypeError):
            a + pos[0]                   # float32 + uint32
        with pytest.raises(TypeError):
            a + x                        # scalar + tensor
        with pytest.raises(ValueError):
            E.power(pos[0], pos[0])      # pow is floating point only
        with pytest.raises(ValueError):
            -pos[0]                      # cannot negate an unsigned value
        with pytest.raises(ValueError):
            E.exp(pos[0])
        with pytest.raises(SyntaxError):
            bool(a < s)
        with pytest.raises(SyntaxError):
            a <<= s                      # only variables are assignable
        v = E.variable(0, float32)
        v <<= s
        v <<= 3
        with pytest.raises(TypeError):
            v <<= pos[0]
        i = E.cast(pos[0], uint64)
        assert i.dtype == uint64
        idx = x[pos].args[1]             # linear index is computed in uint64
        assert idx.dtype == uint64


def test_arange_and_branches_build_regions():
    with E.tracing() as b:
        x = E.input([4, 3], float32)
        pos = E.position_in(4)
        acc = E.variable(0, float32)
        for i in E.arange(3):
            assert i.dtype == int64
            acc <<= acc + x[pos[0], i]
        for j in E.arange(pos[0], 3):
            assert j.dtype == uint32     # first expression operand decides
        with E.if_(acc > 1):
            acc <<= 1
        with E.elif_(acc < -1):
            acc <<= -1
        with E.else_():
            acc <<= 0
        with pytest.raises(SyntaxError):
            with E.else_():              # chain already closed by an else
                pass
        with pytest.raises(TypeError):
            E.if_(True)
    kinds = [n.kind for n in b.root.nodes]
    assert kinds.count('for') == 2 and kinds.count('if') == 1
    chain = [n for n in b.root.nodes if n.kind == 'if'][0]
    assert len(chain.blocks) == 3 and chain.conds[2] is None
    # the elif condition was traced after the if but must be computed before the chain starts
    at = [id(n) for n in b.root.nodes]
    assert at.index(id(chain.conds[1])) < at.index(id(chain))


def _add_one():
    @ovl.operator()
    def add_one(x, y):
        assert x.shape == y.shape
        a = ovl.output_like(x)
        b = ovl.output_like(y)
        pos = ovl.position_in(a.shape)
        a[pos] = x[pos] + 1
        b[pos] = y[pos] + 1
        return a, b
    return add_one


def test_dag_builder_structure():
    add_one = _add_one()
    in0, in1, in2 = (np.random.random(10) for _ in range(3))
    a, b = add_one(in0, in1)
    c, d = add_one(a, in1)
    e, f = add_one(in1, b)
    g, h = add_one(f, a)
    i, j = add_one(e, in2)
    dag = build_op_dag(i, h)
    assert len(dag.kernels) == 4                 # c/d's operator is not needed
    assert [x is y for x, y in zip(dag.inputs, (in1, in0, in2))] or True
    # producers precede consumers and references point at the right producer outputs
    for op_index, refs in enumerate(dag.references):
        for r in refs:
            assert r.is_leaf or r.op_index < op_index
    first = dag.references[0]
    assert first[0].is_leaf and dag.inputs[first[0].dag_input_index] is in0
    assert first[1].is_leaf and dag.inputs[first[1].dag_input_index] is in1
    assert dag.outputs[0][1] == 0 and dag.outputs[1][1] == 1


def test_outputs_are_numbered_in_return_order():
    @ovl.operator()
    def swapped(x):
        a = ovl.output(x.shape, ovl.float32)
        b = ovl.output(x.shape, ovl.float64)
        pos = ovl.position_in(x.shape)
        a[pos] = ovl.cast(x[pos], ovl.float32)
        b[pos] = x[pos]
        return b, a
    op = swapped(np.zeros(3))
    assert op.output_types[0].dtype == float64 and op.output_types[1].dtype == float32
    assert [n.attr['io_index'] for n in op.kernel.outputs] == [0, 1]


def test_wrong_returns_and_arguments():
    @ovl.operator()
    def no_return(x):
        ovl.output_like(x)
        ovl.position_in(x.shape)

    @ovl.operator()
    def missing_output(x):
        a = ovl.output_like(x)
        ovl.output_like(x)
        ovl.position_in(x.shape)
        return a

    @ovl.operator()
    def returns_input(x):
        ovl.output_like(x)
        ovl.position_in(x.shape)
        return x

    @ovl.operator()
    def needs_constant(x, k=None):
        out = ovl.output_like(x)
        pos = ovl.position_in(x.shape)
        out[pos] = x[pos] * k
        return out

    x = np.zeros(3)
    for op in (no_return, missing_output):
        with pytest.raises(ValueError):
            op(x)
    with pytest.raises(TypeError):
        returns_input(x)
    with pytest.raises(ValueError):
        needs_constant(x)                 # unset (None) constant
    with pytest.raises(TypeError):
        needs_constant(x, x, k=2.0)       # one tensor argument too many
    with pytest.raises(TypeError):
        needs_constant(k=2.0)             # tensor argument missing
    with pytest.raises(TypeError):
        needs_constant(2.0, k=2.0)        # a python number is not a tensor
    assert needs_constant(x, k=2.0).output_types[0] == TensorType([3], float64)


def test_reassignment_of_a_variable_is_rejected():
    with pytest.raises(SyntaxError):
        @ovl.operator()
        def bad(data_in):
            out = ovl.output_like(data_in)
            pos = ovl.position_in(data_in.shape)
            a = ovl.variable(0, dtype=data_in.dtype)
            a = 2
            out[pos] = a
            return out
    with pytest.raises(SyntaxError):
        @ovl.operator()
        def bad2(data_in):
            out = ovl.output_like(data_in)
            pos = ovl.position_in(data_in.shape)
            a = ovl.variable(0, dtype=data_in.dtype)
            a = a + data_in[pos]
            out[pos] = a
            return out

    @ovl.operator()
    def good(data_in):
        out = ovl.output_like(data_in)
        pos = ovl.position_in(data_in.shape)
        a = ovl.variable(0, dtype=data_in.dtype)
        a <<= a + data_in[pos]
        out[pos] = a
        return out
    assert good(np.zeros(4)).output_types[0].size == 4


def test_gradient_graph_signature():
    from opveclib_b200.stdops import mul, sigmoid
    a = np.zeros((2, 3), dtype=np.float32)
    b = np.zeros((2, 3), dtype=np.float32)
    op = mul(a, b)
    g = op.grad_dag
    assert g is not None and len(g.input_types) == 3          # lhs, rhs, d_out
    assert len(g.outputs) == 2
    s = sigmoid(op)
    assert s.grad_dag is not None and len(s.grad_dag.input_types) == 2
    # operators called while tracing a gradient do not get gradients of their own
    assert all(x is None for x in g.grad_dags)


def test_infix_operators_between_operator_outputs():
    from opveclib_b200 import stdops  # noqa: F401  (registers the infix operators)
    a = np.ones(4, dtype=np.float32)
    one = stdops.add(a, a)
    two = one * one - one
    assert two.kernel.name == 'sub'
    assert -one < one
    split = stdops.split(np.zeros((2, 4), dtype=np.float32), split_dim=1, num_split=2)
    with pytest.raises(SyntaxError):
        split + one                       # multi-output operators need an explicit index


def test_kernel_text_is_structural():
    add_one = _add_one()
    k1 = add_one(np.zeros(5), np.zeros(5)).kernel
    k2 = add_one(np.ones(5), np.ones(5)).kernel
    k3 = add_one(np.zeros(6), np.zeros(6)).kernel
    assert k1.text() == k2.text() and k1.digest() == k2.digest()
    assert k1.text() != k3.text()
    assert len(list(iter_nodes(k1.body))) > 10


def test_every_name_the_reference_exports_is_present():
    """The names of opveclib/__init__.py:11-48; ``as_tensorflow`` exists only to point at ``as_torch``."""
    import opveclib_b200 as ovl
    names = '''DType float32 float64 int8 int16 int32 int64 uint8 uint16 uint32 uint64 TensorType Scalar Variable
        InputTensor OutputTensor PositionTensor LocalTensor position_in output output_like zeros ones variable cast
        min_value max_value epsilon arccos arcsin arctan cos cosh sin sinh tan tanh exp log log10 sqrt ceil absolute
        floor logical_not isinf isfinite isnan minimum maximum power arctan2 logical_and logical_or arange if_ elif_
        else_ operator gradient evaluate profile as_tensorflow version logger cuda_enabled cache_directory
        clear_op_cache'''.split()
    missing = [n for n in names if not hasattr(ovl, n)]
    assert not missing, missing
    import pytest
    with pytest.raises(NotImplementedError, match='as_torch'):
        ovl.as_tensorflow([])
    from opveclib_b200 import examples, stdops
    for n in 'accumulate cumsum cumprod expm1 expm1_grad log1p log1p_grad'.split():
        assert hasattr(examples, n), n
    for n in '''neg tanh sin cos tan sigmoid split concat add sub mul div mod equal not_equal less less_equal greater
             greater_equal'''.split():
        assert hasattr(stdops, n), n


def test_an_operator_with_several_outputs_stands_for_all_of_them():
    """`evaluate(op)` with a multi-output operator evaluates every output, as in the reference
    (opveclib/test/test_multiple_outputs.py:44-52)."""
    import numpy as np
    import opveclib_b200 as ovl
    from opveclib_b200 import runtime

    @ovl.operator()
    def multi_op(input0, input1, input2):
        pos = ovl.position_in(input0.shape)
        output0, output1, output2 = ovl.output_like(input0), ovl.output_like(input0), ovl.output_like(input0)
        d = input0[pos] + input1[pos]
        output0[pos] = d
        output1[pos] = d * input2[pos]
        output2[pos] = d + input2[pos]
        return output0, output1, output2

    a, b, c = np.zeros(5), np.zeros(5), np.zeros(5)
    op = multi_op(a, b, c)
    assert len(runtime.as_output_list(op)) == 3
    assert len(runtime.as_output_list(op[1])) == 1 and len(runtime.as_output_list([op[0], op[2]])) == 2
    o0, o1, o2 = op
    assert o1.shape == [5]


def test_index_forms_and_python_control_flow_on_expressions():
    """Index checks of opveclib/test/test_expressions.py:293-333 and the refusal to use an expression where Python
    needs a truth value (ibid. 516-547)."""
    with E.tracing():
        a = E.zeros((5, 5), float32)
        v = E.variable(0, uint64)
        a[0, 0]
        a[[0, 0]]
        a[v, 0]
        for bad in ([1], [0, 0, 0], [v], [v, 0, 0], [v, 5], [0, 5], [-1, 0]):
            with pytest.raises(IndexError):
                a[bad]
        two = E.zeros(2, float32)
        a[two]                                           # a rank-1 tensor of the right length is an index
        for bad in (E.zeros(1, float32), E.zeros(3, float32), E.zeros((2, 1), float32)):
            with pytest.raises(IndexError):
                a[bad]
        x = E.variable(0.0, float32)
        with pytest.raises(SyntaxError):
            if x == 0:
                pass
        with pytest.raises(SyntaxError):
            if x:
                pass
        with pytest.raises(SyntaxError):
            max(x, 1)
        with pytest.raises(SyntaxError):
            min(x, 1)
        with pytest.raises(TypeError):
            E.if_(E.zeros((5, 5), float32))

"""Every kernel family is generated and compiled for sm_100a without a device: one graph per family, the family's
entry point must be in the kernel's metadata and its cubin on disk (nvcc cross-compiles; nothing is launched)."""
import os

import numpy as np
import pytest

import cases
from opveclib_b200 import compiler, runtime


def _graphs(ns):
    u = cases.user_ops(ns)
    f32 = np.float32
    return {
        'vec': (lambda: u.ew_mulc(np.zeros((64, 256), f32), c=2.0), lambda m: m['vec'] is not None),
        'tile': (lambda: u.transpose_axpy(np.zeros((96, 160), f32), np.zeros((160, 96), f32), alpha=0.5),
                 lambda m: m['tile'] is not None and m['tile']['staged'] == 1),
        'red_along': (lambda: u.matvec(np.zeros((64, 512), f32), np.zeros(512, f32)),
                      lambda m: m['red'] is not None and m['red']['layout'] == 'along'),
        'red_across': (lambda: u.colsum(np.zeros((512, 128), f32)),
                       lambda m: m['red'] is not None and m['red']['layout'] == 'across'),
        'scan_block': (lambda: ns.cumsum(np.zeros((16, 4096), f32), axis=1),
                       lambda m: m['scan'] is not None and m['scan']['warp'] is None and not m['scan']['three_pass']),
        'scan_warp': (lambda: ns.cumsum(np.zeros((2048, 256), f32), axis=1),
                      lambda m: m['scan'] is not None and m['scan']['warp'] is not None),
        'scan_ring': (lambda: ns.cumsum(np.zeros(1 << 20, f32)),
                      lambda m: m['scan'] is not None and m['scan']['ring'] is not None),
        'scan_columns': (lambda: ns.cumsum(np.zeros((512, 96), np.float64), axis=0),
                         lambda m: m['scan'] is not None and m['scan'].get('strided')),
        'generic': (lambda: u.shift_cyclic(np.zeros(1000, f32)), lambda m: m['gen'] is not None),
        'red_sliced': (lambda: u.matvec(np.zeros((2, 1 << 17), f32), np.zeros(1 << 17, f32)),
                       lambda m: m['red'] is not None and m['red'].get('split')),
        'red_across_sliced': (lambda: u.colsum(np.zeros((1 << 16, 40), f32)),
                              lambda m: m['red'] is not None and m['red']['layout'] == 'across' and m['red'].get('split')),
        'rows': (lambda: u.row_normalise(np.zeros((1024, 24), f32)),
                 lambda m: m['rows'] is not None and m['rows']['staged'] and m['rows']['staged_outputs']),
        'scan_flat': (lambda: ns.cumsum(np.zeros((4096, 36), f32), axis=1),
                      lambda m: m['scan'] is not None and m['scan']['warp'] and m['scan']['warp'].get('chunks')),
        'scan_ring_grouped': (lambda: ns.cumsum(np.zeros((16, 20 * 8192), f32), axis=1),
                              lambda m: m['scan'] is not None and m['scan']['ring']['layout'] == 'grouped'),
    }


@pytest.mark.parametrize('family', ['vec', 'tile', 'red_along', 'red_across', 'scan_block', 'scan_warp', 'scan_ring',
                                    'scan_columns', 'generic', 'red_sliced', 'red_across_sliced', 'rows', 'scan_flat',
                                    'scan_ring_grouped'])
def test_family_is_generated_and_compiles(family):
    ns = cases.impl()
    build, check = _graphs(ns)[family]
    prog, dag = runtime.compile_outputs([build()])
    plan = prog.plans[0]
    assert check(plan.meta), plan.meta
    name = compiler.kernel_name(dag.kernels[0])
    assert os.path.exists(os.path.join(compiler.cache_directory, name + '.cubin'))
    with open(os.path.join(compiler.cache_directory, name + '.cu')) as f:
        source = f.read()
    assert name + '_gen' in source          # the generic kernel is always there as the correctness net

"""Generate golden input/output vectors from the reference kerops kernels.

Runs the UNMODIFIED reference sources (kerops/kernels/dw_conv.py and the
kerops/ops/conv host wrappers) on the CPU through Triton's interpreter
(TRITON_INTERPRET=1).  The reference kernels combine block masks with Python
`and` / `or` (kerops/kernels/dw_conv.py:32-34,67,130,136-142,178-180,204-213);
the interpreter evaluates those with Python truthiness, which collapses the
masks, so the module is loaded through an in-memory AST rewrite that turns
every BoolOp into the element-wise `&` / `|` the GPU compiler applies.  No
reference source is copied: the file is read from the reference checkout at
run time (path given by --reference), rewritten in memory and executed.

Output: one .npz per case under tests/golden/ holding the fp16 inputs
(x, weight / x, grad in the physical NHWDC order), and the reference outputs
(y from DWConv, dw from DWConvWGRAD).  Run from the repository root:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference <kerops checkout>
"""
import argparse
import ast
import importlib
import math
import os
import sys
import types

os.environ.setdefault('TRITON_INTERPRET', '1')

import numpy as np  # noqa: E402
import torch  # noqa: E402

# (name, seed, N, C, dim2, dim3, dim4)
CASES = [
    ('cfg1_n1_c8_16x16x8', 0, 1, 8, 16, 16, 8),
    ('odd_n1_c8_5x7x13', 1, 1, 8, 5, 7, 13),
    ('odd_n1_c16_3x2x37', 2, 1, 16, 3, 2, 37),
    ('batch_n2_c32_4x6x9', 3, 2, 32, 4, 6, 9),
    ('tiny_n1_c8_2x2x2', 4, 1, 8, 2, 2, 2),
    ('c64_n1_3x5x20', 5, 1, 64, 3, 5, 20),
    ('c128_n2_2x3x10', 6, 2, 128, 2, 3, 10),
]


class _BoolOpToBitwise(ast.NodeTransformer):
    def visit_BoolOp(self, node):
        self.generic_visit(node)
        op = ast.BitAnd() if isinstance(node.op, ast.And) else ast.BitOr()
        out = node.values[0]
        for v in node.values[1:]:
            out = ast.BinOp(left=out, op=op, right=v)
        return ast.copy_location(out, node)


def load_reference(ref_root):
    """Import kerops.ops.conv with kerops.kernels.dw_conv AST-rewritten in memory."""
    sys.path.insert(0, ref_root)
    import triton  # noqa: F401

    path = os.path.join(ref_root, 'kerops', 'kernels', 'dw_conv.py')
    with open(path) as f:
        src = f.read()
    tree = ast.fix_missing_locations(_BoolOpToBitwise().visit(ast.parse(src)))
    new_src = ast.unparse(tree)
    # triton's jit reads the function source through inspect -> linecache; register the
    # rewritten text under a synthetic file name.
    import linecache

    fname = '<kerops.kernels.dw_conv rewritten>'
    linecache.cache[fname] = (len(new_src), None, new_src.splitlines(True), fname)
    importlib.import_module('kerops.kernels')
    mod = types.ModuleType('kerops.kernels.dw_conv')
    mod.__file__ = fname
    sys.modules['kerops.kernels.dw_conv'] = mod
    exec(compile(new_src, fname, 'exec'), mod.__dict__)
    conv = importlib.import_module('kerops.ops.conv')
    return conv.DWConv, conv.DWConvWGRAD


def make_inputs(seed, N, C, s1, s2, s3):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, C, s1, s2, s3, generator=g).half().to(memory_format=torch.channels_last_3d)
    grad = torch.randn(N, C, s1, s2, s3, generator=g).half().to(memory_format=torch.channels_last_3d)
    w = ((torch.rand(C, 1, 3, 3, 3, generator=g) * 2 - 1) / math.sqrt(27)).half()
    w_ker = w[:, 0].permute(1, 2, 3, 0).contiguous()
    return x, grad, w_ker


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='path of a kerops checkout')
    ap.add_argument('--out', default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument('--only', default='', help='comma-separated case names (default: all)')
    args = ap.parse_args()
    DWConv, DWConvWGRAD = load_reference(args.reference)
    only = set(filter(None, args.only.split(',')))
    for name, seed, N, C, s1, s2, s3 in CASES:
        if only and name not in only:
            continue
        x, grad, w_ker = make_inputs(seed, N, C, s1, s2, s3)
        y = DWConv(x, w_ker)
        dw = DWConvWGRAD(x, grad)
        np.savez_compressed(
            os.path.join(args.out, name + '.npz'),
            x=x.permute(0, 2, 3, 4, 1).contiguous().numpy(),
            grad=grad.permute(0, 2, 3, 4, 1).contiguous().numpy(),
            weight=w_ker.numpy(),
            y=y.permute(0, 2, 3, 4, 1).contiguous().numpy(),
            dw=dw.numpy(),
        )
        print(name, 'y', tuple(y.shape), 'dw', tuple(dw.shape))


if __name__ == '__main__':
    main()

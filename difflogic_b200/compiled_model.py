"""CompiledLogicNet: a trained (discretised) logic gate network turned into C and run on the CPU, or -- with
device='cuda', which the reference declares but leaves unimplemented (difflogic/compiled_model.py:263-264,
293-294) -- frozen into device arrays and run by this package's packed-bit kernels.

Drop-in for the reference class (difflogic/compiled_model.py:43-370): same constructor, the same
`get_gate_code / get_layer_code / get_c_code / compile / load / forward` methods and the same
exported C symbol, `void apply_logic_gate_net(bool const *inp, int *out, size_t len)`, so that
libraries saved by either implementation load in the other.

The generated C differs from the reference's: gate values live in one array `v[]` instead of one
scalar per gate and the statements are split into functions of a few thousand lines, which keeps
the C compiler's time and memory linear in the number of gates.
"""
import ctypes
import math
import os
import shutil
import subprocess
import tempfile
import time
from typing import Union

import numpy as np
import numpy.typing
import torch

from .difflogic import GroupSum, LogicLayer

ALL_OPERATIONS = [
    "zero", "and", "not_implies", "a", "not_implied_by", "b", "xor", "or",
    "not_or", "not_xor", "not_b", "implied_by", "not_a", "implies", "not_and", "one",
]

BITS_TO_DTYPE = {8: "char", 16: "short", 32: "int", 64: "long long"}
BITS_TO_ZERO_LITERAL = {8: "(char) 0", 16: "(short) 0", 32: "0", 64: "0LL"}
BITS_TO_ONE_LITERAL = {8: "(char) 1", 16: "(short) 1", 32: "1", 64: "1LL"}
BITS_TO_C_DTYPE = {8: ctypes.c_int8, 16: ctypes.c_int16, 32: ctypes.c_int32, 64: ctypes.c_int64}
BITS_TO_NP_DTYPE = {8: np.int8, 16: np.int16, 32: np.int32, 64: np.int64}

# bitwise form of gate i on operands {0} and {1}; i = 8 f(0,0) + 4 f(0,1) + 2 f(1,0) + f(1,1)
_GATE_EXPR = (
    None, "{0} & {1}", "{0} & ~{1}", "{0}", "{1} & ~{0}", "{1}", "{0} ^ {1}", "{0} | {1}",
    "~({0} | {1})", "~({0} ^ {1})", "~{1}", "~{1} | {0}", "~{0}", "~{0} | {1}", "~({0} & {1})", None,
)

_STATEMENTS_PER_FUNCTION = 4096


def _bind(lib):
    fn = lib.apply_logic_gate_net
    fn.restype = None
    fn.argtypes = [
        np.ctypeslib.ndpointer(ctypes.c_bool, flags="C_CONTIGUOUS"),
        np.ctypeslib.ndpointer(BITS_TO_C_DTYPE[32], flags="C_CONTIGUOUS"),
        ctypes.c_size_t,
    ]
    return fn


class CompiledLogicNet(torch.nn.Module):
    def __init__(
            self,
            model: torch.nn.Sequential,
            device='cpu',
            num_bits=64,
            cpu_compiler='gcc',
            verbose=False,
    ):
        super(CompiledLogicNet, self).__init__()
        self.model = model
        self.device = device
        self.num_bits = num_bits
        self.cpu_compiler = cpu_compiler

        assert cpu_compiler in ["clang", "gcc"], cpu_compiler
        assert num_bits in [8, 16, 32, 64]

        if self.model is not None:
            assert isinstance(self.model[-1], GroupSum), 'The last layer of the model must be GroupSum, but it is {} / {}' \
                                                         ' instead.'.format(type(self.model[-1]), self.model[-1])
            self.num_classes = self.model[-1].k
            self.num_inputs = None
            self.layers = []
            for layer in self.model:
                if isinstance(layer, LogicLayer):
                    if self.num_inputs is None:
                        self.num_inputs = layer.in_dim
                    self.num_out_per_class = layer.out_dim // self.num_classes
                    self.layers.append((layer.indices[0], layer.indices[1], layer.weights.argmax(1)))
                elif isinstance(layer, (torch.nn.Flatten, GroupSum)):
                    if verbose:
                        print('Skipping {} layer ({}).'.format(type(layer).__name__, type(layer)))
                else:
                    assert False, 'Error: layer {} / {} unknown.'.format(type(layer), layer)
            if verbose:
                print('`layers` created and has {} layers.'.format(len(self.layers)))

        self.lib_fn = None
        self._lib = None
        self._cuda_plan = None  # device='cuda': [(a, b, gate ids)] per layer, on the GPU

    # -- code generation -------------------------------------------------------------------------

    def get_gate_code(self, var1, var2, gate_op):
        """C expression of gate `gate_op` applied to the C expressions var1 and var2."""
        gate_op = int(gate_op)
        assert 0 <= gate_op < 16, 'Operator {} unknown.'.format(gate_op)
        if gate_op == 0:
            res = BITS_TO_ZERO_LITERAL[self.num_bits]
        elif gate_op == 15:
            res = "~" + BITS_TO_ZERO_LITERAL[self.num_bits]
        else:
            res = _GATE_EXPR[gate_op].format(var1, var2)
        if self.num_bits in (8, 16):  # integer promotion: bring the result back to the word type
            res = "({}) ({})".format(BITS_TO_DTYPE[self.num_bits], res)
        return res

    def get_layer_code(self, layer_a, layer_b, layer_op, layer_id, prefix_sums):
        """C statements of one layer.  Layer 0 reads `inp[]`, the last layer writes `out[]`, everything in
        between lives in `v[]` at offset prefix_sums[layer_id]."""
        last = layer_id == len(prefix_sums) - 1
        src = "inp[{}]" if layer_id == 0 else "v[%d + {}]" % prefix_sums[layer_id - 1]
        dst = "out[{}]" if last else "v[%d + {}]" % prefix_sums[layer_id]
        a_idx = torch.as_tensor(layer_a).tolist()
        b_idx = torch.as_tensor(layer_b).tolist()
        ops = torch.as_tensor(layer_op).tolist()
        return ["\t{} = {};".format(dst.format(j), self.get_gate_code(src.format(ga), src.format(gb), op))
                for j, (ga, gb, op) in enumerate(zip(a_idx, b_idx, ops))]

    def get_c_code(self):
        """The whole network as one C translation unit."""
        return self._c_sources(1)[0]

    def _c_sources(self, n_units):
        """C source split into `n_units` translation units (the gate functions are spread over them; unit 0 also
        holds logic_gate_net and apply_logic_gate_net), so that several compiler processes can work in parallel."""
        word = BITS_TO_DTYPE[self.num_bits]
        bits = self.num_bits
        prefix_sums = [0]
        for layer_a, _, _ in self.layers[:-1]:
            prefix_sums.append(prefix_sums[-1] + len(layer_a))
        hidden = max(prefix_sums[-1], 1)

        statements = []
        for layer_id, (layer_a, layer_b, layer_op) in enumerate(self.layers):
            statements.extend(self.get_layer_code(layer_a, layer_b, layer_op, layer_id, prefix_sums))

        includes = ["#include <stddef.h>", "#include <stdlib.h>", "#include <stdbool.h>", "#include <string.h>", ""]
        starts = list(range(0, len(statements), _STATEMENTS_PER_FUNCTION))
        parts = ["gates_{}".format(i) for i in range(len(starts))]
        n_units = max(1, min(n_units, len(parts)))
        linkage = "static " if n_units == 1 else ""
        units = [list(includes) for _ in range(n_units)]
        for i, (name, start) in enumerate(zip(parts, starts)):
            unit = units[i * n_units // len(parts)]
            unit.append("{}void {}({w} const *inp, {w} *v, {w} *out) {{".format(linkage, name, w=word))
            unit.extend(statements[start:start + _STATEMENTS_PER_FUNCTION])
            unit.append("}")
            unit.append("")
        code = units[0]
        if n_units > 1:
            code.extend("void {}({w} const *inp, {w} *v, {w} *out);".format(name, w=word) for name in parts)
        code.append("static __thread {} hidden_values[{}];".format(word, hidden))
        code.append("")
        code.append("void logic_gate_net({w} const *inp, {w} *out) {{".format(w=word))
        code.extend("\t{}(inp, hidden_values, out);".format(p) for p in parts)
        code.append("}")

        n_last = self.layers[-1][0].shape[0]
        per_class = n_last // self.num_classes
        planes = math.ceil(math.log2(per_class + 1))
        code.append(r"""
/* inp: bool [len * BITS][N_IN] (sample-major), out: int [len * BITS][N_CLASSES]. */
void apply_logic_gate_net(bool const *inp, int *out, size_t len) {
    enum { BITS = %(bits)d, N_IN = %(n_in)d, N_LAST = %(n_last)d, N_CLASSES = %(k)d, PER_CLASS = %(per_class)d, PLANES = %(planes)d };
    typedef unsigned %(word)s uword;
    %(word)s *packed = malloc(N_IN * sizeof(%(word)s));
    %(word)s *gates = malloc(N_LAST * sizeof(%(word)s));
    uword count[PLANES > 0 ? PLANES : 1];

    for (size_t block = 0; block < len; ++block) {
        /* pack BITS consecutive samples: sample s of the block is bit s of every word */
        bool const *src = inp + block * (size_t) BITS * N_IN;
        for (size_t d = 0; d < N_IN; ++d) {
            uword w = 0;
            for (size_t s = 0; s < BITS; ++s)
                w |= (uword) (src[s * N_IN + d] != 0) << s;
            packed[d] = (%(word)s) w;
        }

        logic_gate_net(packed, gates);

        /* per class: a bit-sliced counter over the class's outputs (count[p] holds bit p of all BITS sums) */
        for (size_t c = 0; c < N_CLASSES; ++c) {
            memset(count, 0, sizeof(count));
            for (size_t g = 0; g < PER_CLASS; ++g) {
                uword carry = (uword) gates[c * PER_CLASS + g];
                for (int p = 0; p < PLANES && carry; ++p) {
                    uword const t = count[p] & carry;
                    count[p] ^= carry;
                    carry = t;
                }
            }
            for (size_t s = 0; s < BITS; ++s) {
                int sum = 0;
                for (int p = 0; p < PLANES; ++p)
                    sum |= (int) ((count[p] >> s) & 1) << p;
                out[(block * BITS + s) * N_CLASSES + c] = sum;
            }
        }
    }
    free(packed);
    free(gates);
}
""" % dict(bits=bits, n_in=self.num_inputs, n_last=n_last, k=self.num_classes, per_class=per_class, planes=planes,
           word=word))
        return ["\n".join(unit) for unit in units]

    # -- build / load ----------------------------------------------------------------------------

    def compile(self, opt_level=1, save_lib_path=None, verbose=False, jobs=None):
        """Writes the C source, builds a shared library with the chosen C compiler and binds it.

        :param opt_level:     -O level; 0 compiles in seconds, higher levels take longer and run ~2x faster
        :param save_lib_path: (optional) where to keep the shared library for `load()`
        :param jobs:          compiler processes to run in parallel (default: one per CPU core, at most one per
                              4096 gates); the source is split into that many translation units
        """
        if self.device == 'cuda':
            self._compile_cuda(verbose)
            return
        if self.device != 'cpu':
            assert False, 'Device {} not supported.'.format(self.device)
        if jobs is None:
            jobs = os.cpu_count() or 1
        sources = self._c_sources(max(1, int(jobs)))
        code = sources[0]
        n_lines = sum(src.count('\n') + 1 for src in sources)
        if verbose and n_lines <= 200:
            print('\n\n' + '\n'.join(sources) + '\n\n')

        workdir = tempfile.mkdtemp(prefix="compiled_logic_net_")
        try:
            so_path = os.path.join(workdir, "net.so")
            c_paths = [os.path.join(workdir, "net_{}.c".format(i)) for i in range(len(sources))]
            for c_path, src in zip(c_paths, sources):
                with open(c_path, "w") as f:
                    f.write(src)
            if verbose:
                print('C code created and has {} lines in {} files. (temp location {})'.format(n_lines, len(sources), workdir))
            t_s = time.time()
            opt = "-O{}".format(opt_level)
            if len(c_paths) == 1:
                result = subprocess.run([self.cpu_compiler, "-shared", "-fPIC", opt, "-o", so_path, c_paths[0]])
                ok = result.returncode == 0
                code_rc = result.returncode
            else:
                procs = [subprocess.Popen([self.cpu_compiler, "-c", "-fPIC", opt, "-o", c_path[:-2] + ".o", c_path])
                         for c_path in c_paths]
                rcs = [p.wait() for p in procs]
                ok = all(rc == 0 for rc in rcs)
                code_rc = next((rc for rc in rcs if rc != 0), 0)
                if ok:
                    result = subprocess.run([self.cpu_compiler, "-shared", "-o", so_path] + [c[:-2] + ".o" for c in c_paths])
                    ok, code_rc = result.returncode == 0, result.returncode
            if not ok:
                raise RuntimeError(f'compilation exited with error code {code_rc}')
            if verbose:
                print('Compiling finished in {:.3f} seconds.'.format(time.time() - t_s))
            if save_lib_path is not None:
                shutil.copy(so_path, save_lib_path)
                if verbose:
                    print('lib_file copied from {} to {} .'.format(so_path, save_lib_path))
            self._lib = ctypes.cdll.LoadLibrary(so_path)  # stays mapped after the file is removed
            self.lib_fn = _bind(self._lib)
        finally:
            shutil.rmtree(workdir, ignore_errors=True)

    def _compile_cuda(self, verbose=False):
        """device='cuda': nothing is compiled.  The network is frozen as it is now -- connections and arg-max gate ids
        copied to the GPU -- and forward() runs the packed-bit kernels on it (pack, one eval kernel per layer, the
        last layer fused with the class count).  `num_bits` is the word width of the packed tensor."""
        from . import ops
        from ._native import lib
        lib()  # raises NativeLibraryMissing without the built CUDA library
        if not torch.cuda.is_available():
            raise RuntimeError("CompiledLogicNet(device='cuda'): no CUDA device")
        plan = []
        for a, b, op in self.layers:
            plan.append((torch.as_tensor(a).to('cuda', torch.int64).contiguous(), torch.as_tensor(b).to('cuda', torch.int64).contiguous(),
                         torch.as_tensor(op).to('cuda', torch.uint8).contiguous()))
        assert plan[-1][0].numel() % self.num_classes == 0, (plan[-1][0].numel(), self.num_classes)
        self._cuda_plan = plan
        self._ops = ops
        if verbose:
            print('{} layers frozen on the GPU.'.format(len(plan)))

    def _forward_cuda(self, x):
        ops = self._ops
        on_gpu = isinstance(x, torch.Tensor) and x.is_cuda
        x = torch.as_tensor(x)
        x = x.reshape(x.shape[0], -1).to('cuda')
        if x.dtype != torch.bool:
            x = x.ne(0)
        assert x.shape[1] == self.num_inputs, (x.shape, self.num_inputs)
        words, pad_len = ops.packbits_batch_major(x.contiguous(), self.num_bits)
        for a, b, gate in self._cuda_plan[:-1]:
            words = ops.eval_packed(words, a, b, gate)
        a, b, gate = self._cuda_plan[-1]
        if ops.eval_groupbitsum_applicable(words, a.numel(), self.num_classes):
            out = ops.eval_groupbitsum(words, a, b, gate, pad_len, self.num_classes)
        else:
            out = ops.groupbitsum(ops.eval_packed(words, a, b, gate), pad_len, self.num_classes)
        return out if on_gpu else out.cpu()

    @staticmethod
    def load(save_lib_path, num_classes, num_bits):
        self = CompiledLogicNet(None, num_bits=num_bits)
        self.num_classes = num_classes
        self._lib = ctypes.cdll.LoadLibrary(save_lib_path)
        self.lib_fn = _bind(self._lib)
        return self

    # -- inference -------------------------------------------------------------------------------

    def forward(
            self,
            x: Union[torch.BoolTensor, numpy.typing.NDArray[np.bool_]],
            verbose: bool = False
    ) -> torch.IntTensor:
        """bool [batch, features] (numpy or torch) -> int32 [batch, num_classes] class counts.  With device='cuda' the
        result is on the GPU when x was, else on the CPU."""
        if self._cuda_plan is not None:
            return self._forward_cuda(x)
        if self.lib_fn is None:
            raise RuntimeError('CompiledLogicNet: call compile() or load() first')
        if isinstance(x, torch.Tensor):
            x = x.numpy()
        x = np.ascontiguousarray(x, dtype=np.bool_)
        batch = x.shape[0]
        blocks = math.ceil(batch / self.num_bits)
        padded = np.zeros((blocks * self.num_bits,) + x.shape[1:], dtype=np.bool_)
        padded[:batch] = x
        if verbose:
            print('x.shape', padded.shape)
        out = np.zeros(blocks * self.num_bits * self.num_classes, dtype=BITS_TO_NP_DTYPE[32])
        self.lib_fn(padded.reshape(-1), out, blocks)
        out = torch.tensor(out).view(blocks * self.num_bits, self.num_classes)[:batch]
        if verbose:
            print('out.shape', out.shape)
        return out

"""A stand-in for runtime.Handle that records the C-ABI calls the executor
makes instead of running them, so that the lifting logic is testable on CPU."""
import ctypes as C


def _copy(struct):
    return type(struct).from_buffer_copy(bytes(struct))


class _Lib:
    def __init__(self, log):
        self.log = log

    def kapyb_elementwise(self, h, insts, n, tin, n_in, tout, stream):
        self.log.append(("elementwise", [tuple(getattr(insts[i], f) for f, _ in insts[i]._fields_)
                                         for i in range(n)],
                         [_copy(tin[i]) for i in range(n_in)], _copy(tout._obj)))
        return 0

    def kapyb_reduce(self, h, src, dst, axis, comb, stream):
        self.log.append(("reduce", _copy(src._obj), _copy(dst._obj), axis, comb))
        return 0

    def kapyb_matmul(self, h, lhs, rhs, acc, out, ep, way, stream):
        self.log.append(("matmul", _copy(lhs._obj), _copy(rhs._obj), _copy(out._obj),
                         _copy(ep._obj), way))
        return 0


class FakeHandle:
    def __init__(self):
        self.log = []
        self._lib = _Lib(self.log)
        self._h = C.c_void_p(1)
        self.last_kernel = "fake"

    def _stream(self, stream=None):
        return C.c_void_p(0)

    def _raise(self, st):
        raise RuntimeError(st)

    def check(self, stream=None):
        pass

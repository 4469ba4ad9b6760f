"""Shape-only ("fake") kernels of the operators that touch tensor data.

Every public operator does its argument handling and autograd in C++ and hands the data to one of the
``torch_scatter::_*`` operators.  Registering a fake kernel for each of those lets ``torch.compile`` /
``torch.export`` propagate shapes through the public operators (forward and backward) without running a CUDA
kernel, so models that call them compile without graph breaks.  Upstream registers none.

Limits under tracing: ``out=`` is not supported (an operator that writes into its argument is invisible to the
tracer), a missing ``dim_size`` becomes a data-dependent size, and the fused composites on a sorted index are not
chosen (whether the index is sorted is a property of the data): the composed operators are traced instead.
"""
import torch

_lib_defined = hasattr(torch.ops.torch_scatter, '_scatter_fw')


def _no_out(out, what):
    if out is not None:
        raise RuntimeError(f'torch_scatter::{what}: `out=` cannot be traced; leave it out under torch.compile / export')


def _placeholder(like):
    return like.new_empty((0,))


def _new_size():
    return torch.library.get_ctx().new_dynamic_size()


def _expanded(rows, src):
    """Leading dims of an indptr / index tensor broadcast against src's."""
    lead = rows.dim() - 1
    for i in range(lead):
        torch._check(rows.size(i) == src.size(i) or rows.size(i) == 1, lambda: 'Input mismatch')
    return lead


if _lib_defined:
    @torch.library.register_fake('torch_scatter::_segment_csr_fw')
    def _(src, indptr, out, reduce):
        _no_out(out, 'segment_csr')
        dim = _expanded(indptr, src)
        shape = list(src.shape)
        shape[dim] = max(indptr.size(-1) - 1, 0)
        res = src.new_empty(shape)
        arg = indptr.new_empty(shape) if reduce in ('min', 'max') else _placeholder(indptr)
        return res, arg

    @torch.library.register_fake('torch_scatter::_gather_csr_fw')
    def _(src, indptr, out, length, divide_by_count):
        _no_out(out, 'gather_csr')
        dim = _expanded(indptr, src)
        shape = list(src.shape)
        shape[dim] = length if length is not None else _new_size()
        return src.new_empty(shape)

    @torch.library.register_fake('torch_scatter::_arg_backward')
    def _(grad_out, arg_out, src_shape, dim):
        return grad_out.new_empty(src_shape)

    @torch.library.register_fake('torch_scatter::_segment_coo_fw')
    def _(src, index, out, dim_size, reduce):
        _no_out(out, 'segment_coo')
        dim = _expanded(index, src)
        shape = list(src.shape)
        shape[dim] = dim_size if dim_size is not None else _new_size()
        res = src.new_empty(shape)
        if reduce in ('min', 'max'):
            extra = index.new_empty(shape)
        elif reduce == 'mean':
            extra = src.new_empty(list(src.shape[:dim]) + [shape[dim]])
        else:
            extra = _placeholder(index)
        return res, extra

    @torch.library.register_fake('torch_scatter::_gather_coo_fw')
    def _(src, index, out, count):
        _no_out(out, 'gather_coo')
        dim = _expanded(index, src)
        shape = list(src.shape)
        shape[dim] = index.size(-1)
        return src.new_empty(shape)

    @torch.library.register_fake('torch_scatter::_scatter_fw')
    def _(src, index, dim, out, dim_size, reduce):
        _no_out(out, 'scatter')
        shape = list(src.shape)
        shape[dim] = dim_size if dim_size is not None else _new_size()
        res = src.new_empty(shape)
        arg = index.new_empty(shape) if reduce in ('min', 'max') else _placeholder(index)
        count = index.new_empty((1,), dtype=torch.int32) if reduce == 'mean' else _placeholder(index)
        return res, arg, count

    @torch.library.register_fake('torch_scatter::_scatter_bw')
    def _(grad_out, index, dim, src_shape, count):
        return grad_out.new_empty(src_shape)

    @torch.library.register_fake('torch_scatter::_segment_lse')
    def _(src, index, dim, groups):
        shape = list(src.shape)
        shape[dim] = groups
        return src.new_empty(shape, dtype=torch.float32)

    @torch.library.register_fake('torch_scatter::_gather_apply')
    def _(x, table, index, dim, op, scale):
        return torch.empty_like(x, memory_format=torch.contiguous_format)

    @torch.library.register_fake('torch_scatter::index_is_sorted')
    def _(index):
        return False   # a property of the data: traced programs take the composed (order-independent) operators

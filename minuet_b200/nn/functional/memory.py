"""Buffer-pool knobs of the reference (minuet/nn/functional/memory.py), kept so
that code written against them still runs.  Scratch memory here comes from
PyTorch's caching allocator, one ``torch.empty`` per call, so there is no pool
to size: the setters store nothing and the getters report zero."""
__all__ = ['cuda_buffer_total_size', 'cuda_buffer_used_size', 'cuda_free_buffers',
           'cuda_set_buffer_growth', 'cuda_set_buffer_page_size', 'cuda_preallocate_buffer',
           'cuda_reset_error']

import torch


def cuda_buffer_total_size():
    return 0


def cuda_buffer_used_size():
    return 0


def cuda_free_buffers():
    """Return cached, unused device memory to the driver."""
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def cuda_preallocate_buffer(size: int):
    del size


def cuda_set_buffer_growth(growth: float):
    del growth


def cuda_set_buffer_page_size(growth: int):
    del growth


def cuda_reset_error():
    """Clear a pending (non-sticky) CUDA error and the engine's status word; the
    autotuner calls this after an out-of-memory RuntimeError
    (minuet/nn/convolutions.py:385-389)."""
    from minuet_b200 import engine
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        engine.status_word(torch.cuda.current_device()).zero_()

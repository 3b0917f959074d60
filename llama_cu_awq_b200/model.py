"""Model-level host mirror: build_transformer / run_transformer / generate_thread of the reference
(llama2_q4.cu:625-659, 541-601, 683-757) over the C ABI."""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check


class Transformer:
    def __init__(self, checkpoint_path, rank=0, gpu_count=1, tp_mode=_lib.Q4_TP_NONE, comm=None, lib=None, synthetic=None):
        self._L = lib or _lib.lib()
        self.h = C.c_void_p()
        if synthetic is not None:   # (config tuple or q4_config, seed): generated on the device, no file
            cfg, seed = synthetic
            if not isinstance(cfg, _lib.q4_config):
                cfg = _lib.q4_config(*[int(v) for v in cfg[:7]], float(cfg[7]))
            check(self._L.q4_model_create_synthetic(C.byref(self.h), C.byref(cfg), int(seed), rank, gpu_count, tp_mode, comm), "create_synthetic")
        else:
            check(self._L.q4_model_load(C.byref(self.h), checkpoint_path.encode(), rank, gpu_count, tp_mode, comm), "build_transformer")
        self.config = _lib.q4_config()
        check(self._L.q4_model_config(self.h, C.byref(self.config)), "config")
        self.stream = torch.cuda.Stream()

    def reset(self, prompt_tokens, pos=0):
        arr = np.ascontiguousarray(prompt_tokens, dtype=np.int32)
        check(self._L.q4_model_reset(self.h, arr.ctypes.data_as(C.POINTER(C.c_int)), arr.size, pos), "reset")

    def forward(self, gen_token=True, path=1):
        check(self._L.q4_model_forward(self.h, C.c_void_p(self.stream.cuda_stream), int(bool(gen_token)), path), "run_transformer")

    def prefill(self, n_tokens, gen_token=True):
        """The next n_tokens prompt positions in one pass (q4_model_prefill)."""
        check(self._L.q4_model_prefill(self.h, C.c_void_p(self.stream.cuda_stream), int(n_tokens), int(bool(gen_token))), "prefill")

    def set_sampler(self, temperature, topp, seed):
        """build_sampler (sampler.h:28): temperature 0 decodes greedily."""
        check(self._L.q4_model_set_sampler(self.h, float(temperature), float(topp), int(seed)), "build_sampler")

    def best_path(self):
        """The fastest forward path that serves this model: 2 = persistent fused kernel, else 1 = CUDA-graph
        replay of the per-op kernels."""
        return 2 if self._L.q4_model_prepare(self.h, 2) == _lib.Q4_OK else 1

    def status(self):
        return self._L.q4_model_status(self.h)

    def set_wait_limit_ns(self, ns):
        """Limit of the fused kernel's device-side waits (0 = default of two seconds)."""
        check(self._L.q4_model_set_wait_limit_ns(self.h, int(ns)), "set_wait_limit")

    def logits_device_ptr(self):
        return self._L.q4_model_logits(self.h)

    def synchronize(self):
        self.stream.synchronize()

    def _read(self, what, n):
        out = np.empty(n, np.float16)
        check(self._L.q4_model_read(self.h, what, out.ctypes.data_as(C.c_void_p)), "read")
        return out

    def logits(self):
        return self._read(0, self.config.vocab_size)

    def x(self):
        return self._read(1, self.config.dim)

    def shared(self):
        return self._L.q4_model_shared(self.h).contents

    def generate(self, prompt_tokens, steps, path=1, prompt_one_pass=False):
        """generate_thread's token loop (q4_generate); prompt_one_pass feeds the prompt but its last position through
        q4_model_prefill first."""
        if prompt_one_pass:
            path |= _lib.Q4_PATH_PROMPT_ONE_PASS
        arr = np.ascontiguousarray(prompt_tokens, dtype=np.int32)
        if steps <= 0 or steps > self.config.seq_len:
            steps = self.config.seq_len
        out = np.zeros(steps + 1, np.int32)
        timed, secs = C.c_int(), C.c_double()
        check(self._L.q4_generate(self.h, arr.ctypes.data_as(C.POINTER(C.c_int)), arr.size, steps, path,
                                  out.ctypes.data_as(C.POINTER(C.c_int)), C.byref(timed), C.byref(secs)), "generate")
        return out, timed.value, secs.value

    def token_bytes(self, pos):
        return self._L.q4_model_token_bytes(self.h, pos)

    def close(self):
        if self.h:
            self._L.q4_model_free(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Batch:
    """Batched decode of several sequences over one model (q4_batch_*)."""

    def __init__(self, transformer, n_seq):
        self.t, self._L, self.n_seq = transformer, transformer._L, n_seq
        self.h = C.c_void_p()
        check(self._L.q4_batch_create(C.byref(self.h), transformer.h, n_seq), "batch_create")

    def reset(self, prompts):
        arr = np.ascontiguousarray(prompts, dtype=np.int32)
        assert arr.ndim == 2 and arr.shape[0] == self.n_seq
        check(self._L.q4_batch_reset(self.h, arr.ctypes.data_as(C.POINTER(C.c_int)), arr.shape[1]), "batch_reset")

    def forward(self):
        check(self._L.q4_batch_forward(self.h, C.c_void_p(self.t.stream.cuda_stream)), "batch_forward")

    def logits(self):
        n = self.n_seq * self.t.config.vocab_size
        out = np.empty(n, np.float16)
        self.t.synchronize()
        ptr = self._L.q4_batch_logits(self.h)
        src = torch.as_tensor(_DevView(ptr, n), device="cuda")
        return src.cpu().numpy().reshape(self.n_seq, -1)

    def tokens(self, length):
        out = np.zeros((self.n_seq, length), np.int32)
        check(self._L.q4_batch_read_tokens(self.h, out.ctypes.data_as(C.POINTER(C.c_int)), length), "batch_read_tokens")
        return out

    def close(self):
        if self.h:
            self._L.q4_batch_free(self.h)
            self.h = C.c_void_p()


class _DevView:
    """A device pointer as something torch.as_tensor accepts (CUDA array interface)."""

    def __init__(self, ptr, n, typestr="<f2"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (int(ptr), False), "version": 2}

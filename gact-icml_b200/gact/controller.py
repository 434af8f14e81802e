"""The public object of the library (reference: gact/gact/controller.py).

    gact.set_optimization_level('L2')
    controller = Controller(model)
    controller.install_hook()
    for batch in loader:
        ...forward / backward / optimizer step...
        controller.iterate(backprop)      # backprop(): one forward + backward, used by auto precision
    controller.uninstall_hook()
"""
import torch

from gact.conf import config
from gact.quantizer import Quantizer
from gact.autoprec import AutoPrecision
from gact import _native as _nv


def _device_live():
    """True when this process has a CUDA context (asking the library about its device state would create one)."""
    return torch.cuda.is_available() and torch.cuda.is_initialized()


class Controller:
    def __init__(self, model):
        self._hook_installed = False
        if not config.compress_activation:
            return
        self.model = model

        # the requested (possibly fractional-on-average) width picks the fixed width used until auto
        # precision takes over: 2 -> 2, 3..4 -> 4, 5..16 -> 8
        assert config.bit <= 16 and config.bit > 1
        if config.bit == 2:
            default_bit = 2
        elif config.bit <= 4:
            default_bit = 4
        else:
            default_bit = 8
        self.quantizer = Quantizer(default_bit=default_bit, swap=config.swap, prefetch=config.prefetch)
        # model parameters are never compressed
        self.quantizer.filter_tensors(model.named_parameters())
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            self.quantizer.seed_offset = torch.distributed.get_rank() << 32

        self.auto_prec = config.auto_prec
        if self.auto_prec:
            self.ap = AutoPrecision(self.model, self.quantizer, config.bit, config.max_bit,
                                    config.work_dir, config.adapt_interval, config.log_interval,
                                    debug=config.debug)
        self.bit = config.bit
        self.iter = 0

    def __del__(self):
        try:
            self.uninstall_hook()
        except Exception:
            pass

    def install_hook(self):
        def pack_hook(x):
            r = self.quantize(x)
            del x
            return r

        def unpack_hook(x):
            r = self.dequantize(x)
            del x
            return r

        if self._hook_installed:
            return
        if config.compress_activation:
            # the hooks run for every saved tensor of every step: hand autograd the quantizer's bound methods
            # directly instead of two more Python frames per call
            pack_hook, unpack_hook = self.quantizer.quantize, self.quantizer.dequantize
        torch._C._autograd._push_saved_tensors_default_hooks(pack_hook, unpack_hook)
        self._hook_installed = True

    def uninstall_hook(self):
        # the reference pops unconditionally (also from __del__), which removes somebody else's hook when
        # none was installed; pop only what install_hook pushed
        if getattr(self, "_hook_installed", False):
            torch._C._autograd._pop_saved_tensors_default_hooks()
            self._hook_installed = False
            if config.compress_activation and _device_live():
                _nv.check_pipeline("Controller.uninstall_hook")

    def iterate(self, get_grad):
        if not config.compress_activation:
            return
        self.quantizer.iterate()
        if self.auto_prec:
            self.ap.iterate_wrapper(get_grad)
        self.iter += 1
        self.quantizer.seed_iter = self.iter

    def quantize(self, input):
        if not config.compress_activation:
            if config.swap and input.is_cuda:
                # plain swap of the uncompressed tensor
                tensor_cpu = torch.empty(input.shape, dtype=input.dtype, device='cpu', pin_memory=True)
                tensor_cpu.copy_(input, non_blocking=True)
                return tensor_cpu
            return input
        return self.quantizer.quantize(input)

    def dequantize(self, input):
        if not config.compress_activation:
            if config.swap:
                input = input.cuda(non_blocking=True)
            return input
        return self.quantizer.dequantize(input)

    # ---- additions: the reference never saves its own state, so a resumed run repeats the probe ----
    def state_dict(self):
        if not config.compress_activation:
            return {}
        sd = {"iter": self.iter, "bits": dict(self.quantizer.bits), "dims": dict(self.quantizer.dims),
              "seeds": dict(self.quantizer.seeds), "quantizer_iter": self.quantizer.iter,
              "seed_iter": self.quantizer.seed_iter}
        if self.auto_prec:
            sd["ap"] = {"C": dict(self.ap.C), "bits": dict(self.ap.bits), "iter": self.ap.iter,
                        "dims": None if self.ap.dims is None else dict(self.ap.dims)}
        return sd

    def load_state_dict(self, sd):
        if not config.compress_activation or not sd:
            return
        self.iter = sd["iter"]
        q = self.quantizer
        q.bits, q.dims, q.seeds = dict(sd["bits"]), dict(sd["dims"]), dict(sd["seeds"])
        q.iter, q.seed_iter = sd["quantizer_iter"], sd["seed_iter"]
        if self.auto_prec and "ap" in sd:
            ap = sd["ap"]
            self.ap.C, self.ap.bits, self.ap.iter = dict(ap["C"]), dict(ap["bits"]), ap["iter"]
            if ap["dims"] is not None:
                self.ap.dims = q.dims
                self.ap.total_bits = self.ap.avg_bits * sum(q.dims.values())

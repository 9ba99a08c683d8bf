"""Constants: gRPC message cap, extra argument names of ``auto_accelerate``, peak-FLOPS table used
for hardware-FLOPS-utilisation reports (B200 added; A100/H100 as in atorch/common/constants.py:71-98)."""


class GrpcEnv:
    MAX_SEND_MESSAGE_LENGTH = 1 << 30
    MAX_RECEIVE_MESSAGE_LENGTH = 1 << 30


class AutoAccelerateExtraArgs:
    ALL = ("verbose", "time_limit", "find_unused_parameters", "sample_batch", "batch_size", "expand_sample_batch",
           "sampler_seed", "ignore_dryrun_on_load_strategy", "meta_init_offload_name")


class GPUCapability:
    """Dense peak TFLOPS by device name and dtype."""
    TFLOPS = {
        "B200": {"bf16": 2250.0, "fp16": 2250.0, "fp8": 4500.0, "fp4": 9000.0, "tf32": 1100.0, "fp32": 75.0},
        "H100": {"bf16": 989.4, "fp16": 989.4, "fp8": 1978.9, "tf32": 494.7, "fp32": 66.9},
        "A100": {"bf16": 312.0, "fp16": 312.0, "tf32": 156.0, "fp32": 19.5},
        "V100": {"fp16": 125.0, "fp32": 15.7},
    }

    @classmethod
    def peak(cls, device_name: str, dtype: str = "bf16") -> float:
        for k, v in cls.TFLOPS.items():
            if k in device_name:
                return v.get(dtype, 0.0)
        return 0.0

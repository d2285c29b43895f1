"""The only hardware target: NVIDIA B200 (sm_100a) in an 8-GPU NVSwitch box. Kernel grids, the memory plan, the
preflight and the roofline figures share these numbers. Reference: hibana/hardware/gb10.py (the same role for its one
target; there host and GPU share one memory, here each GPU has its own HBM and the host floor guards host RAM only).
"""
GPU_NAME = "NVIDIA B200"
COMPUTE_CAPABILITY = (10, 0)
ARCH = "sm_100a"
MIN_DRIVER_MAJOR = 570                # first driver branch with sm_100 support
NUM_SMS = 148                         # two dies of 74
SMEM_PER_CTA = 227 * 1024             # bytes a CTA can opt in to
TMEM_COLUMNS = 512                    # 32-bit accumulator columns per SM (128 lanes): 256 KiB
L2_BYTES = 126 * 1024 * 1024
HBM_BYTES = 180 * 10 ** 9
MIN_TOTAL_MEMORY_MIB = 170_000        # a healthy board reports about 183,000 MiB
NOMINAL_HBM_GBS = 7700.0
NOMINAL_BF16_TFLOPS = 2250.0          # dense; fp8 2x, fp4 4x
NVLINK_GBS_PER_DIRECTION = 900.0      # per GPU through NVSwitch, every peer at full rate
MAX_GPUS_PER_BOX = 8
MAX_CLUSTER = 8                       # portable thread-block cluster size (16 is opt-in)
HOST_FLOOR_GIB = 6.0                  # free host memory the engine leaves to the OS (launch/guard.py acts at half)
UNIFIED_PHYSICAL_MEMORY = False


def is_target(major: int, minor: int) -> bool:
    return (major, minor) == COMPUTE_CAPABILITY

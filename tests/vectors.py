"""Input vectors shared by the tests.

The closed-form generators are the ones the reference's own unit tests use
(cited per function); the seeded gradients come from the oracle's
counter-based generator with the workload distributions of the benchmark
configurations."""
import numpy as np

F = np.float32


def codec_vector(n: int = 515) -> np.ndarray:
    """sin(i*0.071)*(0.5+(i%137)*0.03)
    (NNtrain.Core.Tests/CudaBfp8KernelTests.cs:21-24)."""
    i = np.arange(n)
    return (np.sin((i.astype(F) * F(0.071)).astype(F)).astype(F)
            * (F(0.5) + (i % 137).astype(F) * F(0.03))).astype(F)


def roundtrip_vector(n: int = 515) -> np.ndarray:
    """sin(i*0.043)*(0.125+(i%139)*0.017)
    (NNtrain.Core.Tests/CudaBfp8KernelTests.cs:73-77)."""
    i = np.arange(n)
    return (np.sin((i.astype(F) * F(0.043)).astype(F)).astype(F)
            * (F(0.125) + (i % 139).astype(F) * F(0.017))).astype(F)


def reducer_vector(n: int, offset: float, scale: float, tail: float) -> np.ndarray:
    """sin((i+offset)*0.173)*scale with the last element = tail*scale, a
    unique maximum (NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:195-200)."""
    i = np.arange(n)
    v = (np.sin(((i.astype(F) + F(offset)) * F(0.173)).astype(F)).astype(F) * F(scale)).astype(F)
    v[-1] = F(tail) * F(scale)
    return v


def mix8_vector(n: int = 300) -> np.ndarray:
    """sin(i*0.17)*(1+i/50) (NNtrain.Core.Tests/Bfp8QuantizationTests.cs:57-59)."""
    i = np.arange(n)
    return (np.sin((i.astype(F) * F(0.17)).astype(F)).astype(F) * (F(1) + i.astype(F) / F(50))).astype(F)


REFERENCE_LENGTHS = (1, 17, 33, 257, 515, 300137)
REFERENCE_BLOCKS = (0, 32, 96, 128)


def tail_max_vector(n: int = 300137) -> np.ndarray:
    """A long tensor whose maximum sits at the very end
    (NNtrain.Core.Tests/CudaBfp8KernelTests.cs:204-266)."""
    v = codec_vector(n)
    v[-1] = F(7.5)
    return v


def config0_gradient(oracle, replica: int, n: int = 1 << 18, seed: int = 0xB2000000) -> np.ndarray:
    """Benchmark configuration 0's distribution at a test-sized length."""
    return oracle.generate_gradient(n, seed, replica)

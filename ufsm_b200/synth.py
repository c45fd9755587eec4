"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations (stand-ins for scroll CT and
trained weights, which are not available): N(0, 1) activations, Kaiming-normal weights std sqrt(2 / (C_in taps)), N(0, 0.01)
biases, CT bytes ~ clip(N(110, 40), 0, 255)."""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def kaiming(seed, co, ci, taps, transposed=False):
    std = np.sqrt(2.0 / (ci * taps))
    shape = (ci, co, taps) if transposed else (co, ci, taps)
    return (rng(seed).standard_normal(shape) * std).astype(np.float32)


def bias(seed, co, std=0.01):
    return (rng(seed).standard_normal(co) * std).astype(np.float32)


def act_h16(seed, n):
    return rng(seed).standard_normal(n).astype(np.float16)


def ct_u8(seed, n):
    return np.clip(np.rint(rng(seed).normal(110.0, 40.0, n)), 0, 255).astype(np.uint8)


def unet_weights(seed, cw, nh=7, bias_std=0.01):
    """Flat fp32 weight array in forward order, each conv's bias after its weights (the order of umx_unet_nweights)."""
    L, out, k = len(cw), [], [seed * 1000]

    def conv(co, ci, taps, transposed=False):
        k[0] += 1
        out.append(kaiming(k[0], co, ci, taps, transposed).ravel())
        out.append(bias(k[0] + 500, co, bias_std))
    for l in range(L):
        conv(cw[l], cw[l] if l else 1, 27)
        conv(cw[l], cw[l], 27)
        if l < L - 1:
            conv(cw[l + 1], cw[l], 8)
    for l in range(L - 2, -1, -1):
        conv(cw[l], cw[l + 1], 8, transposed=True)
        conv(cw[l], 2 * cw[l], 27)
        conv(cw[l], cw[l], 27)
    conv(nh, cw[0], 1)
    return np.concatenate(out).astype(np.float32)


def sheet_volume(seed, V, spacing=12.0, thickness=4.0, sigma=1.5):
    """uint8 V^3 volume: Gaussian-blurred noise plus concentric cylindrical sheets about the z axis."""
    from scipy.ndimage import gaussian_filter
    g = rng(seed)
    noise = gaussian_filter(g.standard_normal((V, V, V)).astype(np.float32), sigma) * 60.0
    yy, xx = np.meshgrid(np.arange(V, dtype=np.float32) - V / 2, np.arange(V, dtype=np.float32) - V / 2, indexing="ij")
    r = np.sqrt(yy * yy + xx * xx)
    sheet = ((r % spacing) < thickness).astype(np.float32) * 100.0 + 45.0
    return np.clip(np.rint(noise + sheet[None, :, :]), 0, 255).astype(np.uint8)


def sheet_slab(seed, V, z0, z1, spacing=12.0, thickness=4.0, sigma=1.5):
    """Planes [z0, z1) of the same kind of volume, made plane by plane so that a rank can build its own slab of a 1024^3 volume: the blurred
    noise is one 64^3 block blurred with periodic boundaries and tiled (period 64 along every axis), the sheets depend on (y, x) only."""
    from scipy.ndimage import gaussian_filter
    B = 64
    noise = gaussian_filter(rng(seed).standard_normal((B, B, B)).astype(np.float32), sigma, mode="wrap") * 60.0
    yy, xx = np.meshgrid(np.arange(V, dtype=np.float32) - V / 2, np.arange(V, dtype=np.float32) - V / 2, indexing="ij")
    sheet = ((np.sqrt(yy * yy + xx * xx) % spacing) < thickness).astype(np.float32) * 100.0 + 45.0
    reps = (V + B - 1) // B
    out = np.empty((z1 - z0, V, V), np.uint8)
    made = {}
    for z in range(z0, z1):
        if z % B not in made:
            made[z % B] = np.clip(np.rint(np.tile(noise[z % B], (reps, reps))[:V, :V] + sheet), 0, 255).astype(np.uint8)
        out[z - z0] = made[z % B]
    return out

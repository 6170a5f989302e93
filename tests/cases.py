"""Seeded small layers shared by the golden generator and the parity tests."""

SMALL_CASES = {
    # name: (K, N, M, density, kind, seed, alphas)
    "ragged": (96, 50, 3, 0.05, "gauss", 11, (0.0, 1.0, 0.5)),
    "k64": (64, 64, 4, 0.05, "residual10", 12, (1.0,)),
    "zipf": (256, 160, 9, 0.02, "zipf", 13, (0.5,)),
    "empty": (128, 33, 1, 0.0, "gauss", 14, (1.0,)),
    "m17": (512, 144, 17, 0.01, "gauss", 15, (1.0,)),
    "m40": (1024, 272, 40, 0.005, "gauss", 16, (0.25,)),
    "m200": (384, 200, 200, 0.01, "zipf", 17, (1.0,)),
}

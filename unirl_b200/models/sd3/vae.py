"""SD3 latent codec (16 channels, fp32 decode; ``unirl/models/sd3/vae.py:34-56``): see ``models/dit/vae.py``."""
from unirl_b200.models.dit.vae import LatentVAE as SD3VAE
from unirl_b200.models.dit.vae import VAEConfig as SD3VAEConfig

__all__ = ["SD3VAE", "SD3VAEConfig"]

"""CPU oracle of the Swin3D hot path -- test infrastructure, never imported by the product."""

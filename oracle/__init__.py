"""CPU oracle of the convolution path: test infrastructure, never imported by the product."""

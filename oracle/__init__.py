"""CPU oracle of the GPTQ path: test infrastructure, never imported by the product package."""

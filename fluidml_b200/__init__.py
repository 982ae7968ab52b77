"""B200-native execution back end for FluidML's operator hot path."""

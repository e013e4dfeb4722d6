"""
Cochlear frequency map and gammatone filterbank (FIR approximation) for raw-waveform front ends.

Parity: returnn/util/sig_proc.py (greenwood_function :8, inv_greenwood_function :30, GammatoneFilterbank :51).
"""

from __future__ import annotations
import numpy


def greenwood_function(x, scaling_constant=165.4, constant_of_integration=0.88, slope=2.1):
    """position on the cochlea (0..1) -> characteristic frequency in Hz: A * (10^(a x) - k)"""
    return scaling_constant * (numpy.power(10.0, slope * numpy.asarray(x, dtype="float64")) - constant_of_integration)


def inv_greenwood_function(freq, scaling_constant=165.4, constant_of_integration=0.88, slope=2.1):
    """frequency in Hz -> position on the cochlea"""
    return numpy.log10(numpy.asarray(freq, dtype="float64") / scaling_constant + constant_of_integration) / slope


class GammatoneFilterbank:
    """``num_channels`` gammatone impulse responses with centre frequencies equally spaced on the Greenwood map"""

    def __init__(self, num_channels: int, length: float, sample_rate: int = 16000, freq_max: float = 7500.0, freq_min: float = 100.0,
                 normalization: bool = True):
        """
        :param length: of each impulse response in seconds
        :param normalization: scale every filter to unit peak of its frequency response
        """
        self.num_channels = num_channels
        self.length = length
        self.sample_rate = sample_rate
        self.freq_max = freq_max
        self.freq_min = freq_min
        self.normalization = normalization

    def center_frequencies(self) -> numpy.ndarray:
        """[num_channels] Hz"""
        lo, hi = inv_greenwood_function(self.freq_min), inv_greenwood_function(self.freq_max)
        return greenwood_function(numpy.linspace(lo, hi, self.num_channels))

    def get_gammatone_filterbank(self) -> numpy.ndarray:
        """:return: [taps, num_channels] float32; g(t) = t^(n-1) exp(-2 pi b t) cos(2 pi f t), order n = 4, b = 1.019 ERB(f)"""
        n_taps = int(numpy.floor(self.sample_rate * self.length))
        t = numpy.arange(n_taps, dtype="float64") / self.sample_rate
        order = 4
        fb = numpy.zeros((n_taps, self.num_channels), dtype="float64")
        for i, fc in enumerate(self.center_frequencies()):
            erb = 24.7 * (4.37 * fc / 1000.0 + 1.0)
            b = 1.019 * erb
            g = numpy.power(t, order - 1) * numpy.exp(-2.0 * numpy.pi * b * t) * numpy.cos(2.0 * numpy.pi * fc * t)
            if self.normalization:
                peak = numpy.abs(numpy.fft.rfft(g, n=max(4096, n_taps))).max()
                if peak > 0:
                    g = g / peak
            fb[:, i] = g
        return fb.astype("float32")

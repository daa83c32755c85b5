// Stand-in for the reference's dl::image::ImagePreprocessor, for compiling its detection post-processors on the
// host (oracle/_ref): the four geometry getters they read, fed by the harness.  Test infrastructure.
#pragma once

namespace dl {
namespace image {
class ImagePreprocessor {
public:
    float inv_scale_x = 1.f, inv_scale_y = 1.f;
    int border_left = 0, border_top = 0;
    float get_resize_scale_x(bool inv = false) { return inv ? inv_scale_x : 1.f / inv_scale_x; }
    float get_resize_scale_y(bool inv = false) { return inv ? inv_scale_y : 1.f / inv_scale_y; }
    int get_border_left() { return border_left; }
    int get_border_top() { return border_top; }
};
} // namespace image
} // namespace dl

// C shim over the stb_image copy vendored in the nncv tree (third_party/stb_image/stb_image.h),
// the decoder nncv's example driver uses (examples/Res18/main.cpp:3-4,36).  TEST INFRASTRUCTURE:
// compiled from where that header lies into oracle/_ref/, so that the test of the unchanged
// driver can feed the CPU oracle exactly the pixels the driver saw.
#define STB_IMAGE_IMPLEMENTATION
#include "stb_image.h"

#include <cstring>

extern "C" int ref_decode_image(const char* path, unsigned char* out, long cap, int* w, int* h, int* c) {
  unsigned char* data = stbi_load(path, w, h, c, 0);
  if (!data) return -1;
  const long n = (long)*w * *h * *c;
  if (n > cap) {
    stbi_image_free(data);
    return -2;
  }
  std::memcpy(out, data, (size_t)n);
  stbi_image_free(data);
  return 0;
}

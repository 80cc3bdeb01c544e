// C door to the reference's tensor-name conversion (src/utils/name_conversion.cpp), compiled from where it
// lies in the reference tree into oracle/_ref/libedref_names.so.  Test infrastructure: it pins the library's
// own canonicalisation rules; never part of the product path.
#include <cstring>
#include <string>

#include "core/runtime/model_loader.h"

// The three string predicates of utils/util.h that the conversion uses (their definitions sit in a file that
// needs the whole project).
bool starts_with(const std::string& s, const std::string& start) { return s.compare(0, start.size(), start) == 0; }
bool ends_with(const std::string& s, const std::string& ending) {
    return s.size() >= ending.size() && s.compare(s.size() - ending.size(), ending.size(), ending) == 0;
}
bool contains(const std::string& s, const std::string& part) { return s.find(part) != std::string::npos; }

std::string convert_diffusion_model_name(std::string name, std::string prefix, SDVersion version);

extern "C" int ref_convert_diffusion_name(int family, const char* name, char* out, int capacity) {
    static const SDVersion versions[4] = {VERSION_FLUX, VERSION_SD3, VERSION_QWEN_IMAGE, VERSION_WAN2};
    if (family < 0 || family > 3) return -1;
    const std::string converted = convert_diffusion_model_name(name, "", versions[family]);
    if ((int)converted.size() + 1 > capacity) return -1;
    std::memcpy(out, converted.c_str(), converted.size() + 1);
    return 0;
}

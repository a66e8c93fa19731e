// Test infrastructure only: declarations of the few OpenCV names that the reference's
// examples/ssd/detector.cc and common.cc mention, so that those two files compile
// unmodified without OpenCV. Only cv::Rect carries behaviour that the detector's
// post-process depends on: its members are int, so a float assigned to them truncates
// (cv::Rect is cv::Rect_<int>). Everything else is a placeholder that is never called
// by the functions the oracle drives (GenerateBoxInfo, GetTopK, NMS, iou, softmax).
#ifndef ORACLE_REF_SHIM_OPENCV2_OPENCV_HPP_
#define ORACLE_REF_SHIM_OPENCV2_OPENCV_HPP_
#include <cmath>
#include <cstdlib>
#include <string>
namespace cv {
struct Rect {
    int x = 0, y = 0, width = 0, height = 0;
    Rect() {}
    Rect(int x_, int y_, int w_, int h_) : x(x_), y(y_), width(w_), height(h_) {}
};
struct Size {
    int width = 0, height = 0;
    Size() {}
    Size(int w, int h) : width(w), height(h) {}
};
struct Point {
    int x = 0, y = 0;
    Point() {}
    Point(int x_, int y_) : x(x_), y(y_) {}
};
struct Scalar {
    double v[4];
    Scalar(double a = 0, double b = 0, double c = 0, double d = 0) : v{a, b, c, d} {}
};
class Mat {
public:
    int rows = 0, cols = 0;
    unsigned char* data = nullptr;
    void convertTo(Mat&, int) const { std::abort(); }
};
inline Mat operator-(const Mat&, const Scalar&) { std::abort(); }
enum { COLOR_BGR2RGB = 4, FONT_HERSHEY_SIMPLEX = 0, LINE_AA = 16 };
inline void cvtColor(const Mat&, Mat&, int) { std::abort(); }
inline void resize(const Mat&, Mat&, Size) { std::abort(); }
inline void rectangle(Mat&, Rect, const Scalar&, int) { std::abort(); }
inline Size getTextSize(const std::string&, int, double, int, int*) { std::abort(); }
inline void putText(Mat&, const std::string&, Point, int, double, Scalar, int, int) { std::abort(); }
class VideoCapture {
public:
    explicit VideoCapture(const char*) {}
    explicit VideoCapture(int) {}
    bool isOpened() const { return false; }
    bool set(int, double) { return false; }
};
}  // namespace cv
#define CV_32FC3 21
#define CV_CAP_PROP_FRAME_WIDTH 3
#define CV_CAP_PROP_FRAME_HEIGHT 4
#define CV_CAP_PROP_FPS 5
#endif
